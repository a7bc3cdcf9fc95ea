#!/usr/bin/env python
"""Benchmark of the SRWM / delta-rule hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

A "step" is one forward + backward pass of the operator over the (rank-local shard of the)
workload's batch -- the backward also sums the per-sample state gradients over the local batch
into the slow-weight gradient bucket -- and, for N > 1, the bucket's NCCL all-reduce (enqueued
behind the backward and overlapped with the next step's forward).  The default workload is the
scale-sweep configuration: SRWM, B=1024 (global, batch-sharded over the ranks), H=16,
d_head=64, L=2048, bf16 activations, fp32 state, run through the layer-level entry points with
the slow weights un-repeated ([1,H,d,.], batch stride 0).  The same run also times the
delta-rule configuration of the sweep (B=512, H=16, d=64, L=8192) and reports it under "delta".

Rank 0 prints ONE JSON line.  ``value`` is whole-job tokens/s (B*L / step time, max over
ranks) with the inputs resident in HBM; ``e2e`` is the same metric through the public
autograd entry point (``self_ref_v0``) with the activations starting in pinned host memory
and the slow-weight gradients read back to the host every step.  ``roofline`` is the HBM
view of the dominant kernel (the metric asks for it), ``roofline_fp32`` its CUDA-core fp32
view (the ceiling that binds); ``parity_spot`` compares two sequences of the last timed step
with the float64 oracle; ``small_configs`` times the two small reference configurations.

``--impl reference`` times the reference math (its per-step PyTorch loop with autograd,
restated in oracle/srwm_oracle.py) on the host CPU cores, on a bounded sample of the
workload (the line's ``config`` names the sample); rank 0 only.  When a GPU and the
reference's own CUDA extensions (built unmodified into oracle/_ref) are present, that arm
also times those kernels inside their valid envelope and reports them under
``ref_cuda_kernels``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "modern-srwm_b200"))

import torch  # noqa: E402

# ---- workloads (the benchmark configurations; inputs are seeded synthetic tensors of those shapes) ----
WORKLOADS = {
    # name: op, B (global), H, L, E, dtype
    "srwm_c5": dict(op="srwm", B=1024, H=16, L=2048, E=64, dtype="bf16"),
    "delta_c5": dict(op="delta", B=512, H=16, L=8192, E=64, dtype="bf16"),
    "srwm_c1": dict(op="srwm", B=4, H=4, L=64, E=16, dtype="f32"),
    "delta_c2": dict(op="delta", B=32, H=8, L=512, E=64, dtype="f32"),
    "srwm_c3op": dict(op="srwm", B=128, H=16, L=128, E=32, dtype="f32"),
    "srwm_c4_learner": dict(op="srwm", B=32, H=8, L=100, E=32, dtype="f32"),
    # small cases for profiler captures (saved activations still exceed the 126 MB L2,
    # and the grid is a whole number of waves: 592 = 148 SMs x 4, 1184 = 148 x 8)
    "srwm_prof": dict(op="srwm", B=37, H=16, L=512, E=64, dtype="bf16"),
    "delta_prof": dict(op="delta", B=74, H=16, L=1024, E=64, dtype="bf16"),
    "srwm_prof32": dict(op="srwm", B=111, H=16, L=512, E=32, dtype="f32"),    # 1776 sequences = 148 x 12
    # the layer-level kernels on the same capture sizes: layer forward (input softmax, shift state,
    # reset mask) + detached-state backward; packed delta forward + backward
    "srwm_layer_prof": dict(op="srwm_layer", B=37, H=16, L=512, E=64, dtype="bf16"),
    "delta_layer_prof": dict(op="delta_packed", B=74, H=16, L=1024, E=64, dtype="bf16"),
}

# CPU sample sizes for the host baseline (same H, E, dtype=fp32 math; fewer sequences/steps)
CPU_SAMPLE = {"srwm": dict(B=4, L=256), "delta": dict(B=4, L=512)}


def algorithmic_bytes(op, E, s, per="fwd+bwd"):
    """Bytes per (sequence, step) that the operator must move (s = bytes per activation
    element), and bytes per sequence for the state."""
    D = 3 * E + 4
    if op in ("srwm", "srwm_layer"):
        fwd = E * s + E * s + (5 * E + 8) * 4              # x read, y write, saved write
        bwd = 2 * E * s + E * s + (5 * E + 8) * 4          # x, dy read, dx write, saved read
        st_f, st_b = 2 * E * D * 4, 2 * E * D * 4          # W0 read + W_L write ; W_L read + dW write
        if op == "srwm_layer":                             # detached backward: k, y_diff, beta; W_y only
            bwd = 2 * E * s + E * s + (2 * E + 4) * 4
            st_f, st_b = 3 * E * D * 4, 3 * E * E * 4
    else:
        fwd = (3 * E + 1) * s + E * s + 2 * E * 4          # q,k,v,beta read, out write, v_old/v_ins write
        bwd = (3 * E + 1) * s + E * s + (3 * E + 1) * s + 2 * E * 4
        st_f, st_b = 2 * E * E * 4, 2 * E * E * 4
        if op == "delta_packed":
            st_f = E * E * 4                               # zero-initialised state is not read
    if per == "fwd":
        return fwd, st_f
    if per == "bwd":
        return bwd, st_b
    return fwd + bwd, st_f + st_b


def algorithmic_flops(op, E):
    """Flops per (sequence, step), forward and backward (FMA = 2)."""
    D = 3 * E + 4
    if op == "srwm_layer":
        return 6 * E * D, 6 * E * E
    n = E * D if op == "srwm" else E * E
    return 6 * n, 14 * n


# CUDA-core fp32 ceiling: SMs x fp32 lanes per SM x 2 flops per FMA x clock
N_SM, FP32_LANES = 148, 128


def fp32_peak_tflops(sm_mhz):
    return N_SM * FP32_LANES * 2 * sm_mhz * 1e6 / 1e12


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as fh:
            d = json.load(fh)
        return float(d["hbm_gbs"]), "measured", float(d.get("sm_max_mhz", 1965.0))
    return 6650.0, "fallback", 1965.0


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.lines = []
        self.proc = None
        self.thr = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thr = threading.Thread(target=self._pump, daemon=True)
        self.thr.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1])); power.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "power_w_max": max(power), "samples": len(sm)}


# ---------------------------------------------------------------------------------------
# CPU reference arm / baseline
# ---------------------------------------------------------------------------------------

def cpu_reference_pass(op, H, E, B, L, seed=0):
    """One forward+backward of the reference math (per-step PyTorch loop, autograd) in fp32
    on the host cores.  Returns seconds."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import srwm_oracle as orc
    g = torch.Generator().manual_seed(seed)
    if op == "srwm":
        x = torch.randn(B, H, L, E, generator=g).requires_grad_()
        std = E ** -0.5
        Ws = [(torch.randn(B, H, E, E, generator=g) * std).requires_grad_() for _ in range(3)]
        Ws.append((torch.randn(B, H, E, 4, generator=g) * std).requires_grad_())
        go = torch.randn(B, H, L, E, generator=g)
        t0 = time.perf_counter()
        out, _ = orc.srwm_loop(x, *Ws, update_last=False)
        (out * go).sum().backward()
        return time.perf_counter() - t0
    Q = torch.softmax(torch.randn(B, H, L, E, generator=g), -1).requires_grad_()
    K = torch.softmax(torch.randn(B, H, L, E, generator=g), -1).requires_grad_()
    V = torch.randn(B, H, L, E, generator=g).requires_grad_()
    Bt = torch.sigmoid(torch.randn(B, H, L, 1, generator=g)).requires_grad_()
    W0 = torch.zeros(B, H, E, E)
    go = torch.randn(B, H, L, E, generator=g)
    t0 = time.perf_counter()
    out, _ = orc.delta_loop(Q, K, V, Bt, W0)
    (out * go).sum().backward()
    return time.perf_counter() - t0


def cpu_baseline(wl, runs=3):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    s = CPU_SAMPLE[wl["op"]]
    cpu_reference_pass(wl["op"], wl["H"], wl["E"], s["B"], s["L"])   # warm-up (thread pool, allocator)
    ts = [cpu_reference_pass(wl["op"], wl["H"], wl["E"], s["B"], s["L"]) for _ in range(runs)]
    t = statistics.median(ts)
    return {"value": s["B"] * s["L"] / t, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"{wl['op']} fwd+bwd, per-step PyTorch loop + autograd, fp32, B={s['B']} H={wl['H']} "
                      f"L={s['L']} d={wl['E']} ({t:.1f} s per pass)"}


def ref_cuda_kernel_timings(steps=20, warmup=5):
    """The reference's own CUDA kernels (oracle/_ref: its two .cu files compiled unmodified for
    sm_100a) forward+backward on cuda:0, on the two configurations inside their valid envelope
    (SRWM d_head 16 within one time chunk; delta rule d 64).  Zero-filled outputs are allocated
    per call exactly as the reference's autograd functions do.  Reference-arm only."""
    if not torch.cuda.is_available():
        return {"unavailable": "no CUDA device in this process"}
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_kernels as ref
    if not ref.available():
        return {"unavailable": "oracle/_ref not built (needs the upstream sources at build time)"}
    dev = torch.device("cuda", 0)
    res = {}
    for name in ("srwm_c1", "delta_c2"):
        wl = WORKLOADS[name]
        B, H, L, E = wl["B"], wl["H"], wl["L"], wl["E"]
        g = torch.Generator(device=dev).manual_seed(11)
        rn = lambda *s: torch.randn(*s, device=dev, generator=g)
        if wl["op"] == "srwm":
            x, go = rn(B, H, L, E), rn(B, H, L, E)
            std = E ** -0.5
            W0 = [rn(B, H, E, E) * std for _ in range(3)] + [rn(B, H, E, 4) * std]
            W = [w.clone() for w in W0]

            def run():
                for a_, b_ in zip(W, W0):
                    a_.copy_(b_)
                _, saved = ref.srwm_forward(x, *W)
                ref.srwm_backward(x, saved, go, *W)
        else:
            Q, K = torch.softmax(rn(B, H, L, E), -1), torch.softmax(rn(B, H, L, E), -1)
            V, Bt, go = rn(B, H, L, E), torch.sigmoid(rn(B, H, L, 1)), rn(B, H, L, E)
            W = torch.zeros(B, H, E, E, device=dev)

            def run():
                W.zero_()
                _, saved = ref.delta_forward(Q, K, V, Bt, W)
                ref.delta_backward(Q, K, V, Bt, saved, go, W)
        for _ in range(warmup):
            run()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            run()
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / steps
        res[name] = {"config": config_of(name, wl, 1)["workload"], "ms_per_step": ms,
                     "tokens_per_s": B * L / (ms * 1e-3)}
    return res


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = WORKLOADS[args.workload]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    s = CPU_SAMPLE[wl["op"]]
    for _ in range(min(args.warmup, 1)):
        cpu_reference_pass(wl["op"], wl["H"], wl["E"], s["B"], s["L"])
    ts = [cpu_reference_pass(wl["op"], wl["H"], wl["E"], s["B"], s["L"], seed=i) for i in range(args.steps)]
    t = sum(ts) / len(ts)
    val = s["B"] * s["L"] / t
    sample = (f"{wl['op']} fwd+bwd, reference per-step PyTorch loop + autograd on the host CPU, fp32, "
              f"B={s['B']} H={wl['H']} L={s['L']} d={wl['E']}")
    # the configuration this arm RAN: a bounded sample of the workload (fewer sequences and steps,
    # same heads and head size), converted to tokens/s
    cfg = {"workload": f"{args.workload} scaled to a CPU sample: {wl['op']} fwd+bwd B={s['B']} H={wl['H']} "
                       f"L={s['L']} d_head={wl['E']} fp32 on {cores} host cores (full workload: B={wl['B']} "
                       f"L={wl['L']} {wl['dtype']} activations)",
           "scaled": True, "global_batch": s["B"], "seq_len": s["L"], "heads": wl["H"], "d_head": wl["E"],
           "full_workload": config_of(args.workload, wl, args.gpus)["workload"],
           "parallelism": "host CPU threads", "l2": "n/a (CPU)"}
    line = {"impl": "reference", "metric": "SRWM/delta fwd+bwd tokens/s", "value": val, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    if not args.no_ref_cuda:
        try:
            line["ref_cuda_kernels"] = ref_cuda_kernel_timings()
        except Exception as exc:   # the CPU line must still be printed
            line["ref_cuda_kernels"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    print(json.dumps(line), flush=True)


def config_of(name, wl, n):
    return {"workload": f"{name}: {wl['op']} fwd+bwd B={wl['B']} H={wl['H']} L={wl['L']} d_head={wl['E']} "
                        f"{wl['dtype']} activations, fp32 state",
            "global_batch": wl["B"], "seq_len": wl["L"], "heads": wl["H"], "d_head": wl["E"],
            "parallelism": f"batch-sharded x{n}" + ("; slow weights un-repeated [1,H,d,.], batch reduction of the "
                                                     "gradients fused into the backward (into one flat bucket), "
                                                     "one NCCL all-reduce per step"
                                                     if wl["op"].startswith("srwm") else ""),
            "l2": "inputs_exceed_l2"}


# ---------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------

class OpBench:
    """Holds device-resident inputs of one workload shard and runs steps through the C ABI."""

    def __init__(self, wl, Bl, device, seed):
        import srwm_b200 as sb
        from srwm_b200 import layer_ops
        from srwm_b200.dist import GradBucket
        self.sb, self.lo, self.wl, self.Bl, self.dev = sb, layer_ops, wl, Bl, device
        H, L, E = wl["H"], wl["L"], wl["E"]
        dt = torch.bfloat16 if wl["dtype"] == "bf16" else torch.float32
        self.dt = dt
        g = torch.Generator(device=device).manual_seed(seed)
        rn = lambda *s: torch.randn(*s, device=device, dtype=torch.float32, generator=g)
        self.launches_per_step = 0
        self.bucket = None
        op = wl["op"]
        if op in ("srwm", "srwm_layer"):
            self.x = self._big_randn((Bl, H, L, E), g, dt)
            self.go = self._big_randn((Bl, H, L, E), g, dt)
            std = E ** -0.5
            # the slow weights stay [1,H,d,.]: the kernels read them with a batch stride of zero
            self.slow = [rn(1, H, E, E) * std for _ in range(3)] + [rn(1, H, E, 4) * std]
            self.bucket = GradBucket([w.shape[1:] for w in self.slow], device)
            if op == "srwm_layer":
                self.shift = [0.05 * std * rn(Bl, H, E, w.shape[-1]) for w in self.slow]
                self.done = torch.rand(Bl, L, device=device, generator=g) < 0.01
        elif op == "delta":
            self.Q = self._big_randn((Bl, H, L, E), g, dt, softmax=True)
            self.K = self._big_randn((Bl, H, L, E), g, dt, softmax=True)
            self.V = self._big_randn((Bl, H, L, E), g, dt)
            self.Bt = torch.sigmoid(rn(Bl, H, L, 1)).to(dt)
            self.go = self._big_randn((Bl, H, L, E), g, dt)
            self.W = torch.zeros(Bl, H, E, E, device=device)
        else:   # delta_packed: the layers' raw slow-net rows [q | k | v | b], time-major
            RS = 3 * E + 1
            raw = self._big_randn((L, Bl, H * RS), g, dt)
            self.rows = raw.view(L, Bl, H, RS).permute(1, 2, 0, 3)
            self.go = self._big_randn((Bl, H, L, E), g, dt)
            self.W = torch.empty(Bl, H, E, E, device=device)
        self.ev = []

    @staticmethod
    def _big_randn(shape, g, dt, softmax=False):
        """Generate N(0,1) (optionally softmax over the feature dim) in batch slices to bound
        the fp32 temporary."""
        out = torch.empty(shape, device=g.device, dtype=dt)
        step = max(1, (1 << 28) // max(1, out[0].numel()))
        for i in range(0, shape[0], step):
            t = torch.randn((min(step, shape[0] - i),) + tuple(shape[1:]), device=g.device, generator=g)
            if softmax:
                t = torch.softmax(t, -1)
            out[i:i + step] = t.to(dt)
        return out

    def step(self, timed=False):
        sb, lo = self.sb, self.lo
        rec = None
        if timed:
            rec = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        op = self.wl["op"]
        if op == "srwm":
            if rec: rec[0].record()
            out, shift_out, saved = lo.srwm_layer_forward(self.x, self.slow, None, None, input_softmax=False)
            if rec: rec[1].record()
            # the backward sums the per-sample dL/dW_0 over the local batch straight into the flat bucket
            # (fused into the kernel's epilogue); the bucket's all-reduce is enqueued behind it and
            # overlaps the next step's forward, so the previous one must have landed before this backward
            self.bucket.wait()
            grads = lo.srwm_layer_backward(self.x, saved, self.go, self.slow, shift_out, None, input_softmax=False,
                                           reduce_into=[self.bucket.view(i) for i in range(4)])
            if rec: rec[2].record()
            self.bucket.all_reduce(async_op=True)
            self.last = (out, grads[0])
            self.launches_per_step = 2
        elif op == "srwm_layer":
            if rec: rec[0].record()
            out, shift_out, saved = lo.srwm_layer_forward(self.x, self.slow, self.shift, self.done, True)
            if rec: rec[1].record()
            gx, gWy = lo.srwm_backward_detached(self.x, saved, self.go, self.slow[0], self.shift[0], self.done, True)
            if rec: rec[2].record()
            self.bucket.wait()
            self.bucket.reduce_into(0, gWy)
            self.bucket.all_reduce(async_op=True)
            self.last = (out, gx)
            self.launches_per_step = 2 + 1
        elif op == "delta":
            self.W.zero_()
            if rec: rec[0].record()
            out, saved = sb.delta_forward(self.Q, self.K, self.V, self.Bt, self.W)
            if rec: rec[1].record()
            grads = sb.delta_backward(self.Q, self.K, self.V, self.Bt, saved, self.go, self.W)
            if rec: rec[2].record()
            self.last = (out, grads[0])
            self.launches_per_step = 2
        else:
            if rec: rec[0].record()
            out, saved = lo.delta_packed_forward(self.rows, self.W, 0.0, True)
            if rec: rec[1].record()
            g = lo.delta_packed_backward(self.rows, saved, self.go, self.W, 0.0)
            if rec: rec[2].record()
            self.last = (out, g[0] if isinstance(g, (tuple, list)) else g)
            self.launches_per_step = 2
        if rec:
            self.ev.append(rec)

    def finish(self):
        """Inside the timed region, after the last step: the pending all-reduce must have landed."""
        if self.bucket is not None:
            self.bucket.wait()

    def kernel_ms(self):
        f = [a.elapsed_time(b) for a, b, _ in self.ev]
        b = [b_.elapsed_time(c) for _, b_, c in self.ev]
        return sum(f) / len(f), sum(b) / len(b)

    def parity_spot(self):
        """Two sequences of the last timed step against the float64 oracle (reverse-time recipe on
        the CPU): max|err| / max|ref| of the forward output and of grad_x.  The streamed tensors are
        bf16 in the sweep configurations, so the bound is bf16 rounding (8e-3), not 1e-4."""
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import srwm_oracle as orc
        wl = self.wl
        if wl["op"] not in ("srwm", "delta"):
            return None
        Bl, H = self.Bl, wl["H"]
        picks = sorted({(0, 0), (Bl - 1, H - 1)})
        out, gx = self.last
        fwd_err = grad_err = 0.0
        for n, h in picks:
            sl = (slice(n, n + 1), slice(h, h + 1))
            c = lambda t: t[sl].detach().double().cpu()
            if wl["op"] == "srwm":
                W0 = [w[:, h:h + 1].double().cpu() for w in self.slow]
                f = orc.srwm_forward_explicit(c(self.x), *W0)
                r = orc.srwm_backward_explicit(c(self.x), f["q"], f["k"], f["beta"], f["y_diff"], f["q_diff"],
                                               f["k_diff"], f["beta_diff"], c(self.go), f["W_y"], f["W_q"],
                                               f["W_k"], f["w_b"])
                ref_out, ref_g = f["out"], r[0]
            else:
                E = wl["E"]
                f = orc.delta_forward_explicit(c(self.Q), c(self.K), c(self.V), c(self.Bt),
                                               torch.zeros(1, 1, E, E, dtype=torch.float64))
                r = orc.delta_backward_explicit(c(self.Q), c(self.K), c(self.V), c(self.Bt), f["v_old"],
                                                f["v_insert"], c(self.go), f["W"])
                ref_out, ref_g = f["out"], r[0]
            fwd_err = max(fwd_err, orc.rel_max(c(out), ref_out))
            grad_err = max(grad_err, orc.rel_max(c(gx), ref_g))
        tol = 8e-3 if wl["dtype"] == "bf16" else 1e-3
        return {"fwd": fwd_err, "grad": grad_err, "sequences": [list(p) for p in picks],
                "metric": "max|err| / max|ref| against the float64 oracle", "tolerance": tol,
                "ok": bool(fwd_err < tol and grad_err < tol)}


def timed_region(fn, steps, warmup, dist_on, device, finish=None):
    import torch.distributed as dist
    for _ in range(warmup):
        fn(False)
    if finish:
        finish()
    torch.cuda.synchronize(device)
    if dist_on:
        dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn(True)
    if finish:
        finish()
    e1.record()
    torch.cuda.synchronize(device)
    if dist_on:
        dist.barrier()
    torch.cuda.synchronize(device)
    ms = e0.elapsed_time(e1)
    if dist_on:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps


def run_e2e(wl, Bl, device, steps, warmup, dist_on):
    """Same metric through the public autograd entry point with host-resident activations.

    Per step: H2D copy of that step's activations from pinned host memory, forward, backward,
    batch reduction of the slow-weight gradients (autograd's repeat-backward), all-reduce,
    and a D2H read of the result, followed by a stream synchronise.  The input pipeline is
    double buffered the way a prefetching data loader is: while step s computes, the copy of
    step s+1's activations runs on a side stream into the other device buffer, so every
    timed step contains exactly one full H2D copy, overlapped with compute."""
    import torch.distributed as dist
    import srwm_b200 as sb
    H, L, E = wl["H"], wl["L"], wl["E"]
    dt = torch.bfloat16 if wl["dtype"] == "bf16" else torch.float32
    g = torch.Generator().manual_seed(7)
    copy_stream = torch.cuda.Stream(device=device)
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    state = {"i": 0}

    def pinned(shape, fill):
        t = torch.empty(shape, dtype=dt).pin_memory()
        chunk = max(1, (1 << 26) // max(1, t[0].numel()))
        for i in range(0, shape[0], chunk):
            t[i:i + chunk] = fill((min(chunk, shape[0] - i),) + tuple(shape[1:])).to(dt)
        return t

    if wl["op"] == "srwm":
        host = [pinned((Bl, H, L, E), lambda s: torch.randn(s, generator=g))]
    else:
        host = [pinned((Bl, H, L, E), lambda s: torch.softmax(torch.randn(s, generator=g), -1)),
                pinned((Bl, H, L, E), lambda s: torch.softmax(torch.randn(s, generator=g), -1)),
                pinned((Bl, H, L, E), lambda s: torch.randn(s, generator=g)),
                pinned((Bl, H, L, 1), lambda s: torch.sigmoid(torch.randn(s, generator=g)))]
    dev = [[torch.empty(h.shape, device=device, dtype=dt) for h in host] for _ in range(2)]
    h2d = sum(h.numel() * h.element_size() for h in host)
    go = torch.randn((Bl, H, L, E), device=device, dtype=dt)

    def prefetch(slot):
        cur = torch.cuda.current_stream(device)
        copy_stream.wait_event(consumed[slot])
        with torch.cuda.stream(copy_stream):
            for d, h in zip(dev[slot], host):
                d.copy_(h, non_blocking=True)
            ready[slot].record(copy_stream)
        del cur

    for ev in consumed:
        ev.record(torch.cuda.current_stream(device))
    prefetch(0)

    if wl["op"] == "srwm":
        std = E ** -0.5
        slow = [(torch.randn(1, H, E, E, device=device) * std).requires_grad_() for _ in range(3)]
        slow.append((torch.randn(1, H, E, 4, device=device) * std).requires_grad_())
        nflat = sum(w.numel() for w in slow)
        hres = torch.empty(nflat, dtype=torch.float32).pin_memory()

        def compute(bufs):
            x = bufs[0].detach().requires_grad_()
            Wb = [w.repeat(Bl, 1, 1, 1) for w in slow]
            out = sb.self_ref_v0(x, *Wb)
            out.backward(go)
            flat = torch.cat([w.grad.reshape(-1) for w in slow])
            if dist_on:
                dist.all_reduce(flat)
            hres.copy_(flat, non_blocking=True)
            for w in slow:
                w.grad = None
    else:
        W = torch.zeros(Bl, H, E, E, device=device)
        hres = torch.empty(Bl * H, dtype=torch.float32).pin_memory()

        def compute(bufs):
            q, k, v, b = (t.detach().requires_grad_() for t in bufs)
            W.zero_()
            out = sb.fast_weight_delta(q, k, v, b, W)
            out.backward(go)
            # per-sequence summary of a gradient as the step's result
            hres.copy_(b.grad.float().sum(dim=(2, 3)).reshape(-1), non_blocking=True)
    d2h = hres.numel() * 4

    def step(_timed):
        slot = state["i"] % 2
        state["i"] += 1
        cur = torch.cuda.current_stream(device)
        prefetch(1 - slot)                 # next step's activations, overlapped with this step
        cur.wait_event(ready[slot])
        compute(dev[slot])
        consumed[slot].record(cur)
        cur.synchronize()                  # the host holds this step's result

    ms = timed_region(step, steps, warmup, dist_on, device)
    copy_stream.synchronize()
    return ms, h2d, d2h


def small_config_timings(device, steps=20, warmup=5):
    """Forward+backward through the plain operator calls at the two small reference
    configurations (the ones the reference's own CUDA kernels are valid at)."""
    res = {}
    for name in ("srwm_c1", "delta_c2"):
        wl = WORKLOADS[name]
        B, H, L, E = wl["B"], wl["H"], wl["L"], wl["E"]
        import srwm_b200 as sb
        g = torch.Generator(device=device).manual_seed(11)
        rn = lambda *s: torch.randn(*s, device=device, generator=g)
        if wl["op"] == "srwm":
            x, go = rn(B, H, L, E), rn(B, H, L, E)
            std = E ** -0.5
            W0 = [rn(B, H, E, E) * std for _ in range(3)] + [rn(B, H, E, 4) * std]
            W = [w.clone() for w in W0]

            def run(_t):
                for a_, b_ in zip(W, W0):
                    a_.copy_(b_)
                _, saved = sb.srwm_forward(x, *W)
                sb.srwm_backward(x, saved, go, *W)
        else:
            Q, K = torch.softmax(rn(B, H, L, E), -1), torch.softmax(rn(B, H, L, E), -1)
            V, Bt, go = rn(B, H, L, E), torch.sigmoid(rn(B, H, L, 1)), rn(B, H, L, E)
            W = torch.zeros(B, H, E, E, device=device)

            def run(_t):
                W.zero_()
                _, saved = sb.delta_forward(Q, K, V, Bt, W)
                sb.delta_backward(Q, K, V, Bt, saved, go, W)
        ms = timed_region(run, steps, warmup, False, device)
        res[name] = {"config": config_of(name, wl, 1)["workload"], "ms_per_step": ms,
                     "tokens_per_s": B * L / (ms * 1e-3)}
    return res


def run_ours(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU fallback for the operators)")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    dist_on = world > 1
    if dist_on:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    from srwm_b200.dist import shard_range
    n = world
    results = {}
    clocks = None
    names = [args.workload] + ([] if args.no_delta or args.workload != "srwm_c5" else ["delta_c5"])
    hbm_peak, peak_kind, sm_max_mhz = load_peaks()
    for name in names:
        wl = WORKLOADS[name]
        lo, hi = shard_range(wl["B"], n, rank)
        Bl = hi - lo
        ob = OpBench(wl, Bl, device, seed=1000 + rank)
        sampler = ClockSampler(local_rank) if (rank == 0 and name == names[0]) else None
        if sampler:
            sampler.start()
        ms = timed_region(ob.step, args.steps, args.warmup, dist_on, device, finish=ob.finish)
        if sampler:
            clocks = sampler.stop()
        fwd_ms, bwd_ms = ob.kernel_ms()
        launches = ob.launches_per_step * args.steps
        spot = ob.parity_spot() if (rank == 0 and n == 1 and not args.no_cpu) else None
        del ob
        torch.cuda.empty_cache()
        e2e_ms, h2d, d2h = (None, 0, 0)
        if not args.no_e2e and wl["op"] in ("srwm", "delta"):
            e2e_ms, h2d, d2h = run_e2e(wl, Bl, device, max(1, args.steps), max(1, min(args.warmup, 3)), dist_on)
            torch.cuda.empty_cache()
        tokens = wl["B"] * wl["L"]
        s = 2 if wl["dtype"] == "bf16" else 4
        seqs_local = Bl * wl["H"]
        per_step, per_seq = algorithmic_bytes(wl["op"], wl["E"], s, "bwd")
        bwd_bytes = seqs_local * (wl["L"] * per_step + per_seq)
        ff, fb = algorithmic_flops(wl["op"], wl["E"])
        achieved = bwd_bytes / (bwd_ms * 1e-3) / 1e9
        bwd_tf = seqs_local * wl["L"] * fb / (bwd_ms * 1e-3) / 1e12
        fwd_tf = seqs_local * wl["L"] * ff / (fwd_ms * 1e-3) / 1e12
        peak32 = fp32_peak_tflops(sm_max_mhz)
        kname = {"srwm": "srwm_bwd_kernel", "srwm_layer": "srwm_bwd_det_kernel", "delta": "delta_bwd_kernel",
                 "delta_packed": "delta_bwd_kernel<PACKED>"}[wl["op"]]
        results[name] = dict(
            wl=wl, ms=ms, tokens_per_s=tokens / (ms * 1e-3), fwd_ms=fwd_ms, bwd_ms=bwd_ms, launches=launches, spot=spot,
            e2e=None if e2e_ms is None else {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s",
                                             "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                                             "ms_per_step": e2e_ms, "steps": max(1, args.steps)},
            # HBM view of the dominant kernel (the metric asks for it).  What binds this kernel is
            # CUDA-core fp32 issue (64-77 flop/B), reported as roofline_fp32.
            roofline={"bound": "fp32_issue", "kernel": kname, "achieved": achieved, "peak": hbm_peak,
                      "unit": "GB/s", "frac": achieved / hbm_peak, "peak_source": f"of {peak_kind}",
                      "traffic": (NCU_BWD_DRAM_BYTES_PER_SEQ_STEP[wl["op"]] * seqs_local * wl["L"]
                                  if wl["E"] == 64 and wl["dtype"] == "bf16" and wl["op"] in NCU_BWD_DRAM_BYTES_PER_SEQ_STEP
                                  else None),
                      "algorithmic_bytes_per_launch": bwd_bytes, "launch_ms": bwd_ms},
            roofline_fp32={"bound": "fp32_issue", "kernel": kname, "achieved": bwd_tf, "peak": peak32,
                           "unit": "TFLOP/s", "frac": bwd_tf / peak32,
                           "peak_source": f"{N_SM} SMs x {FP32_LANES} lanes x 2 x {sm_max_mhz:.0f} MHz (nominal CUDA-core fp32)",
                           "fwd_kernel": {"achieved": fwd_tf, "frac": fwd_tf / peak32, "launch_ms": fwd_ms},
                           "algorithmic_flops_per_launch": seqs_local * wl["L"] * fb})
    if rank == 0:
        main = results[names[0]]
        wl = main["wl"]
        line = {"metric": "SRWM/delta fwd+bwd tokens/s", "value": main["tokens_per_s"], "unit": "tokens/s",
                "n_gpus": n, "steps": args.steps, "warmup": args.warmup, "ms_per_step": main["ms"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f32 state / " + wl["dtype"] + " activations", "data": "synthetic",
                "config": config_of(names[0], wl, n), "roofline": main["roofline"],
                "roofline_fp32": main["roofline_fp32"],
                "kernel_ms": {"fwd": main["fwd_ms"], "bwd": main["bwd_ms"]},
                "gpu_launches": main["launches"], "clocks": clocks}
        if main["e2e"] is not None:
            line["e2e"] = main["e2e"]
        if main["spot"] is not None:
            line["parity_spot"] = main["spot"]
        if n == 1 and not args.no_cpu and wl["op"] in CPU_SAMPLE:
            line["cpu_baseline"] = cpu_baseline(wl)
        for extra in names[1:]:
            r = results[extra]
            line["delta"] = {"value": r["tokens_per_s"], "unit": "tokens/s", "ms_per_step": r["ms"],
                             "config": config_of(extra, r["wl"], n), "roofline": r["roofline"],
                             "roofline_fp32": r["roofline_fp32"],
                             "kernel_ms": {"fwd": r["fwd_ms"], "bwd": r["bwd_ms"]}, "gpu_launches": r["launches"],
                             "e2e": r["e2e"]}
            if r["spot"] is not None:
                line["delta"]["parity_spot"] = r["spot"]
            if n == 1 and not args.no_cpu:
                line["delta"]["cpu_baseline"] = cpu_baseline(r["wl"])
        if n == 1 and args.workload == "srwm_c5" and not args.no_small:
            line["small_configs"] = small_config_timings(device)
        print(json.dumps(line), flush=True)
    if dist_on:
        dist.barrier()
        dist.destroy_process_group()


# DRAM bytes per (sequence, step) of the backward kernels at d_head 64 with bf16 activations,
# from ncu captures of the *_prof workloads (dram__bytes_read.sum + dram__bytes_write.sum
# divided by sequences x steps; profiles/*_d64_bf16_*.txt).  `roofline.traffic` scales this
# to a full launch by the sequence-steps it processes (traffic is streamed once, so it
# grows in proportion).
NCU_BWD_DRAM_BYTES_PER_SEQ_STEP = {"srwm": 1850.2, "delta": 1423.7}


def run_table(args):
    """Operator-level fwd+bwd timings of every configuration (one JSON line each), plus the
    RL actor path: single-step forward calls (L=1, B=48, H=8, d=32) with the state carried,
    through the public entry point under no_grad."""
    import srwm_b200 as sb
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    for name in ("srwm_c1", "delta_c2", "srwm_c3op", "srwm_c4_learner", "srwm_c5", "delta_c5"):
        wl = WORKLOADS[name]
        ob = OpBench(wl, wl["B"], device, seed=1)
        ms = timed_region(ob.step, args.steps, args.warmup, False, device)
        f, b = ob.kernel_ms()
        ff, fb = algorithmic_flops(wl["op"], wl["E"])
        seqs = wl["B"] * wl["H"]
        print(json.dumps({"workload": name, "config": config_of(name, wl, 1)["workload"], "ms_per_step": ms,
                          "tokens_per_s": wl["B"] * wl["L"] / (ms * 1e-3), "fwd_ms": f, "bwd_ms": b,
                          "fwd_tflops": seqs * wl["L"] * ff / (f * 1e-3) / 1e12,
                          "bwd_tflops": seqs * wl["L"] * fb / (b * 1e-3) / 1e12}), flush=True)
        del ob
        torch.cuda.empty_cache()
    # actor path
    B, H, E = 48, 8, 32
    g = torch.Generator(device=device).manual_seed(3)
    x = torch.softmax(torch.randn(B, H, 1, E, device=device, generator=g), -1)
    std = E ** -0.5
    W = [torch.randn(B, H, E, E, device=device, generator=g) * std for _ in range(3)]
    W.append(torch.randn(B, H, E, 4, device=device, generator=g) * std)

    def actor(_timed):
        with torch.no_grad():
            for _ in range(100):
                sb.self_ref_v0(x, *W)

    ms = timed_region(actor, args.steps, args.warmup, False, device)
    print(json.dumps({"workload": "srwm_c4_actor", "config": "SRWM forward only, L=1 B=48 H=8 d=32, state carried, "
                      "100 consecutive calls per step through self_ref_v0 under no_grad",
                      "ms_per_100_calls": ms, "us_per_call": ms * 10.0, "env_steps_per_s": 100 * B / (ms * 1e-3)}),
          flush=True)


def composed_sr_layer(layer, h, state, always_softmax=True):
    """What the reference layers do around the operator (reinforcement_learning/torchbeast/
    layer.py:378-421, supervised_learning/layer.py:156-209), written with torch ops around the
    drop-in ``self_ref_v0`` -- the unfused arm of the layer-level timings."""
    import srwm_b200 as sb
    slen, bsz, _ = h.shape
    H, E = layer.num_head, layer.dim_head
    x = h.reshape(slen, bsz, H, E)
    if always_softmax or getattr(layer, "use_input_softmax", False):
        x = torch.softmax(x, dim=-1)
    x = x.permute(1, 2, 0, 3)
    base = (layer.W_y, layer.W_q, layer.W_k, layer.w_b)
    Ws = [w.repeat(bsz, 1, 1, 1) for w in base]
    if state is not None:
        Ws = [s + w for s, w in zip(state, Ws)]
    out = sb.self_ref_v0(x, *Ws)
    out = out.transpose(1, 2).reshape(bsz, slen, H * E).transpose(0, 1)
    out = layer.drop(layer.out_linear(out))
    out = (layer.layer_norm(h) if getattr(layer, "use_ln", False) else h) + out
    new = tuple(w.detach() - b.detach().repeat(bsz, 1, 1, 1) for w, b in zip(Ws, base))
    return out, new


def run_layer_table(args):
    """Layer-level timings: the fused layer call against the same layer composed from torch
    ops around the drop-in operator (both use this library's kernels for the recurrence)."""
    from srwm_b200.layers import SRWMlayer, SRlayer
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    torch.manual_seed(0)

    def emit(name, cfg, fused, composed, extra=None):
        ms_f = timed_region(fused, args.steps, args.warmup, False, device)
        ms_c = timed_region(composed, args.steps, args.warmup, False, device)
        line = {"workload": name, "config": cfg, "fused_ms": ms_f, "composed_ms": ms_c, "speedup": ms_c / ms_f}
        line.update(extra or {})
        print(json.dumps(line), flush=True)

    # supervised-learning layer, the few-shot model's size: B=128 L=128 H=16 d=32 (dim 512)
    L_, B, H, E = 128, 128, 16, 32
    layer = SRWMlayer(H, E, H * E, 0.0, use_ln=True, use_input_softmax=True).to(device)
    h = torch.randn(L_, B, H * E, device=device)
    tgt = torch.randn(L_, B, H * E, device=device)

    def sl_fused(_t):
        layer.zero_grad(set_to_none=True)
        hh = h.clone().requires_grad_()
        (layer(hh) * tgt).sum().backward()

    def sl_composed(_t):
        layer.zero_grad(set_to_none=True)
        hh = h.clone().requires_grad_()
        (composed_sr_layer(layer, hh, None, always_softmax=False)[0] * tgt).sum().backward()

    emit("srwm_c3_layer", "SRWMlayer fwd+bwd, L=128 B=128 H=16 d=32 dim=512, input softmax, layer norm, fp32",
         sl_fused, sl_composed, {"tokens": L_ * B})

    # reinforcement-learning learner unroll: T=100 B=32 H=8 d=32 (hidden 256), done mask, detached state
    T, B, H, E = 100, 32, 8, 32
    rl = SRlayer(H, E, H * E, 0.0).to(device)
    h = torch.randn(T, B, H * E, device=device)
    tgt = torch.randn(T, B, H * E, device=device)
    done = torch.rand(T, B, device=device) < 0.01
    st0 = [0.05 * torch.randn(B, H, E, E, device=device) for _ in range(3)] + [0.05 * torch.randn(B, H, E, 4, device=device)]

    def rl_fused(_t):
        rl.zero_grad(set_to_none=True)
        hh = h.clone().requires_grad_()
        out, _ = rl.unroll(hh, done, st0)
        (out * tgt).sum().backward()

    def rl_composed(_t):
        rl.zero_grad(set_to_none=True)
        hh = h.clone().requires_grad_()
        st = st0
        outs = []
        for t in range(T):     # reinforcement_learning/torchbeast_procgen/model.py:1180-1197
            nd = (~done[t]).float().view(B, 1, 1, 1)
            st = [nd * s for s in st]
            o, st = composed_sr_layer(rl, hh[t:t + 1], st)
            outs.append(o)
        (torch.cat(outs, 0) * tgt).sum().backward()

    emit("srwm_c4_learner_unroll", "SRlayer learner unroll fwd+bwd, T=100 B=32 H=8 d=32 hidden=256, done mask, "
         "state detached per step: one fused call vs 100 one-step layer calls", rl_fused, rl_composed,
         {"env_steps": T * B})

    # actor: one step, B=48, state carried, no_grad, 100 consecutive calls
    B = 48
    ha = torch.randn(1, B, H * E, device=device)
    sta = [0.05 * torch.randn(B, H, E, E, device=device) for _ in range(3)] + [0.05 * torch.randn(B, H, E, 4, device=device)]

    def actor_fused(_t):
        st = sta
        with torch.no_grad():
            for _ in range(100):
                _, st = rl(ha, st)

    def actor_composed(_t):
        st = sta
        with torch.no_grad():
            for _ in range(100):
                _, st = composed_sr_layer(rl, ha, st)

    emit("srwm_c4_actor_layer", "SRlayer forward, L=1 B=48 H=8 d=32 hidden=256, state carried, no_grad, "
         "100 consecutive layer calls per step", actor_fused, actor_composed, {"calls": 100})

    # ---- model-level: the C3 / C4 stacks (SRWM layer + feed-forward block, twice) -----------------
    import torch.nn as nn

    class FF(nn.Module):   # the residual feed-forward block between the fast-weight layers
        def __init__(self, ff_dim, dim):
            super().__init__()
            self.norm = nn.LayerNorm(dim)
            self.net = nn.Sequential(nn.Linear(dim, ff_dim), nn.ReLU(), nn.Linear(ff_dim, dim))

        def forward(self, x):
            return self.net(self.norm(x)) + x

    # C3: tokens [L=128, B=128, 512] + one-hot(5) -> Linear(517,512) -> 2 x (SRWMlayer(16,32,512) + FF(2048))
    #     -> Linear(512,5), cross-entropy at every position
    L_, B, H, E, D = 128, 128, 16, 32, 512
    c3 = nn.ModuleDict(dict(inp=nn.Linear(D + 5, D), out=nn.Linear(D, 5),
                            sr=nn.ModuleList([SRWMlayer(H, E, D, 0.0) for _ in range(2)]),
                            ff=nn.ModuleList([FF(2048, D) for _ in range(2)]))).to(device)
    feats = torch.randn(L_, B, D, device=device)
    onehot = torch.nn.functional.one_hot(torch.randint(0, 5, (L_, B), device=device), 5).float()
    tok = torch.cat([feats, onehot], -1)
    labels = torch.randint(0, 5, (L_ * B,), device=device)

    def c3_step(fused):
        c3.zero_grad(set_to_none=True)
        hcur = c3["inp"](tok)
        for sr, ff in zip(c3["sr"], c3["ff"]):
            hcur = sr(hcur) if fused else composed_sr_layer(sr, hcur, None, always_softmax=False)[0]
            hcur = ff(hcur)
        torch.nn.functional.cross_entropy(c3["out"](hcur).view(L_ * B, 5), labels).backward()

    emit("srwm_c3_model", "2 x (SRWMlayer(16 heads, d=32, dim 512) + FF(2048)) between Linear(517,512) and "
         "Linear(512,5), cross-entropy, L=128 B=128 fp32, forward+backward", lambda _t: c3_step(True),
         lambda _t: c3_step(False), {"tokens": L_ * B})

    # C4: Linear(257,256) -> 2 x (SRlayer(8 heads, d=32) + FF(512)); learner unroll T=100 B=32 with done
    T, B, H, E, D = 100, 32, 8, 32, 256
    c4 = nn.ModuleDict(dict(inp=nn.Linear(D + 1, D), sr=nn.ModuleList([SRlayer(H, E, D, 0.0) for _ in range(2)]),
                            ff=nn.ModuleList([FF(512, D) for _ in range(2)]))).to(device)
    obs = torch.randn(T, B, D + 1, device=device)
    tgt4 = torch.randn(T, B, D, device=device)
    done4 = torch.rand(T, B, device=device) < 0.01

    def fresh_state(bsz):
        return [[0.05 * torch.randn(bsz, H, E, E, device=device) for _ in range(3)] +
                [0.05 * torch.randn(bsz, H, E, 4, device=device)] for _ in range(2)]

    st4 = fresh_state(B)

    def c4_fused(_t):      # layer by layer over the whole unroll (a layer's state depends on its own inputs only)
        c4.zero_grad(set_to_none=True)
        hcur = c4["inp"](obs)
        for i, (sr, ff) in enumerate(zip(c4["sr"], c4["ff"])):
            hcur, _ = sr.unroll(hcur, done4, st4[i])
            hcur = ff(hcur)
        (hcur * tgt4).sum().backward()

    def c4_composed(_t):   # step by step, as the learner does (torchbeast_procgen/model.py:1180-1197)
        c4.zero_grad(set_to_none=True)
        st = [list(s) for s in st4]
        outs = []
        for t in range(T):
            nd = (~done4[t]).float().view(B, 1, 1, 1)
            hcur = c4["inp"](obs[t:t + 1])
            for i, (sr, ff) in enumerate(zip(c4["sr"], c4["ff"])):
                hcur, st[i] = composed_sr_layer(sr, hcur, [nd * w for w in st[i]])
                hcur = ff(hcur)
            outs.append(hcur)
        (torch.cat(outs, 0) * tgt4).sum().backward()

    emit("srwm_c4_model_learner", "Linear(257,256) + 2 x (SRlayer(8 heads, d=32) + FF(512)), learner unroll T=100 B=32 "
         "with done mask, forward+backward: layer-wise fused unroll vs the step-by-step loop", c4_fused, c4_composed,
         {"env_steps": T * B})

    Ba = 48
    obs_a = torch.randn(1, Ba, D + 1, device=device)
    sta4 = fresh_state(Ba)

    def c4_actor(fused):
        st = [list(s) for s in sta4]
        with torch.no_grad():
            for _ in range(100):
                hcur = c4["inp"](obs_a)
                for i, (sr, ff) in enumerate(zip(c4["sr"], c4["ff"])):
                    hcur, st[i] = sr(hcur, st[i]) if fused else composed_sr_layer(sr, hcur, st[i])
                    hcur = ff(hcur)

    from srwm_b200.graphs import GraphedSRStep
    gstep = GraphedSRStep(list(zip(c4["sr"], c4["ff"])), sta4, obs_a, pre=c4["inp"])

    def c4_actor_graphed(_t):
        for _ in range(100):
            gstep(obs_a)

    ms_g = timed_region(c4_actor_graphed, args.steps, args.warmup, False, device)
    emit("srwm_c4_model_actor", "same stack, actor: one step, B=48, state carried, no_grad, 100 consecutive steps",
         lambda _t: c4_actor(True), lambda _t: c4_actor(False),
         {"calls": 100, "graphed_ms": ms_g, "graphed_us_per_step": ms_g * 10.0,
          "graphed_env_steps_per_s": 100 * Ba / (ms_g * 1e-3)})

    # delta-rule layer of the supervised models: L=512 B=32 H=8 d=64 (dim 512)
    from srwm_b200.layers import FastFFlayer
    import srwm_b200 as sb
    F_ = torch.nn.functional
    L_, B, H, E = 512, 32, 8, 64
    fl = FastFFlayer(H, E, H * E, 0.0).to(device)
    h = torch.randn(L_, B, H * E, device=device)
    tgt = torch.randn(L_, B, H * E, device=device)

    def dl_fused(_t):
        fl.zero_grad(set_to_none=True)
        hh = h.clone().requires_grad_()
        (fl(hh) * tgt).sum().backward()

    def dl_composed(_t):     # supervised_learning/layer.py:66-108 around the drop-in operator
        fl.zero_grad(set_to_none=True)
        hh = h.clone().requires_grad_()
        qkvb = fl.slow_net(fl.layer_norm(hh)).view(L_, B, H, 3 * E + 1)
        q, k, v, b = torch.split(qkvb, (E, E, E, 1), -1)
        b = torch.sigmoid(b)
        q, k, v, b = (t.permute(1, 2, 0, 3) for t in (q, k, v, b))
        q, k = F_.elu(q, 1.0, False) + 1.0, F_.elu(k, 1.0, False) + 1.0
        q, k = q / q.sum(-1, keepdim=True), k / k.sum(-1, keepdim=True)
        W = torch.zeros(B, H, E, E, device=device)
        o = sb.fast_weight_delta(q, k, v, b, W)
        o = hh + fl.out_linear(o.transpose(1, 2).reshape(B, L_, H * E).transpose(0, 1))
        (o * tgt).sum().backward()

    emit("delta_c2_layer", "FastFFlayer fwd+bwd, L=512 B=32 H=8 d=64 dim=512, fp32: packed rows in one call vs "
         "split / elu+1 / sum-norm / sigmoid torch ops around the operator", dl_fused, dl_composed,
         {"tokens": L_ * B})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="srwm_c5", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-delta", action="store_true", help="skip the delta-rule sweep configuration")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-small", action="store_true", help="skip the timings of the two small configurations")
    ap.add_argument("--no-ref-cuda", action="store_true",
                    help="reference arm: do not time the reference's own CUDA kernels")
    ap.add_argument("--table", action="store_true", help="operator-level timings of every configuration")
    ap.add_argument("--layer-table", action="store_true",
                    help="layer-level timings: fused layer call vs torch ops around the operator")
    args = ap.parse_args()
    if args.layer_table:
        run_layer_table(args)
    elif args.table:
        run_table(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
