"""Time the reference's own CUDA kernels (oracle/_ref, built unmodified for sm_100a) against
libsrwm_b200 on the same GPU, forward+backward, inside the reference kernels' valid envelope
(TEST / MEASUREMENT INFRASTRUCTURE; prints one JSON line per case).

    python oracle/time_ref_kernels.py

Cases: SRWM single layer B=4 H=4 L=64 d=16 (the reference's CPU-runnable configuration) and a
larger batch of it; delta rule B=32 H=8 L=512 d=64.  Both sides get the same device tensors;
the reference side includes the zero-filled output allocations its autograd functions make,
ours the uninitialised ones, as in real use.
"""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(HERE, "..", "modern-srwm_b200"))
import ref_kernels as ref  # noqa: E402
import srwm_b200 as sb  # noqa: E402


def timeit(fn, iters=20, warm=5):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def srwm_case(N, H, L, E):
    d = torch.device("cuda", 0)
    g = torch.Generator(device=d).manual_seed(1)
    x = torch.randn(N, H, L, E, device=d, generator=g)
    go = torch.randn(N, H, L, E, device=d, generator=g)
    std = E ** -0.5
    W0 = [torch.randn(N, H, E, E, device=d, generator=g) * std for _ in range(3)]
    W0.append(torch.randn(N, H, E, 4, device=d, generator=g) * std)
    W = [w.clone() for w in W0]

    def run(mod):
        for a, b in zip(W, W0):
            a.copy_(b)
        out, saved = mod.srwm_forward(x, *W)
        mod.srwm_backward(x, saved, go, *W)

    return timeit(lambda: run(ref)), timeit(lambda: run(sb))


def delta_case(N, H, L, E):
    d = torch.device("cuda", 0)
    g = torch.Generator(device=d).manual_seed(2)
    Q = torch.softmax(torch.randn(N, H, L, E, device=d, generator=g), -1)
    K = torch.softmax(torch.randn(N, H, L, E, device=d, generator=g), -1)
    V = torch.randn(N, H, L, E, device=d, generator=g)
    B = torch.sigmoid(torch.randn(N, H, L, 1, device=d, generator=g))
    go = torch.randn(N, H, L, E, device=d, generator=g)
    W = torch.zeros(N, H, E, E, device=d)

    def run_ref():
        W.zero_()
        out, saved = ref.delta_forward(Q, K, V, B, W)
        ref.delta_backward(Q, K, V, B, saved, go, W)

    def run_ours():
        W.zero_()
        out, saved = sb.delta_forward(Q, K, V, B, W)
        sb.delta_backward(Q, K, V, B, saved, go, W)

    return timeit(run_ref), timeit(run_ours)


def main():
    if not ref.available():
        print(json.dumps({"unavailable": "oracle/_ref not built"}))
        return
    for name, fn, shape in [("srwm B=4 H=4 L=64 d=16", srwm_case, (4, 4, 64, 16)),
                            ("srwm B=256 H=16 L=64 d=16", srwm_case, (256, 16, 64, 16)),
                            ("delta B=32 H=8 L=512 d=64", delta_case, (32, 8, 512, 64)),
                            ("delta B=128 H=16 L=1024 d=64", delta_case, (128, 16, 1024, 64))]:
        t_ref, t_ours = fn(*shape)
        N, H, L, E = shape
        print(json.dumps({"case": name, "reference_cuda_ms": round(t_ref, 4), "srwm_b200_ms": round(t_ours, 4),
                          "speedup": round(t_ref / t_ours, 2), "tokens_per_s_ours": N * L / (t_ours * 1e-3),
                          "tokens_per_s_reference_cuda": N * L / (t_ref * 1e-3)}), flush=True)


if __name__ == "__main__":
    main()
