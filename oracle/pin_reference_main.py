"""Pin the oracle against the reference's own self tests and write golden fixtures.

TEST INFRASTRUCTURE.  Runs only in a checkout that has the upstream project next to it
(pass its root with ``--reference``); nothing else in this repository reads that tree.

What it does, for each of the two operators:

1. Reads the reference's package file
   (``supervised_learning/self_ref_v0/__init__.py`` or
   ``supervised_learning/fast_weight/__init__.py``) and executes it *as ``__main__``* on the
   CPU.  Two things are substituted, nothing else:
     * ``torch.utils.cpp_extension.load`` returns a stand-in extension module whose
       ``self_ref_forward/backward`` (``fast_weight_forward/backward``) have the pybind
       signatures of self_ref_v0.cu:1344-1356 (fast_weight_cuda.cu:667-679) and are
       implemented with ``srwm_oracle.*_explicit``;
     * the literal device strings / ``torch.cuda.FloatTensor`` constructors in the test
       body are redirected to the CPU.
   The reference's ``torch.autograd.Function`` classes, its per-step PyTorch loop, its
   ``loss.backward()`` and its assertions (max relative error < 1e-3, eps 1e-6) then run
   unchanged.  If they pass, the oracle's explicit forward/backward agree with the
   reference's autograd loop under the reference's own acceptance metric.
2. Captures the tensors of that run (inputs, the loop's outputs, the loop's autograd
   gradients) and stores them as ``tests/golden/*.pt`` so that the parity tests can replay
   the reference's cases on machines that do not have the reference tree.

Usage:  python oracle/pin_reference_main.py --reference /path/to/modern-srwm
"""
from __future__ import annotations

import argparse
import contextlib
import io
import os
import re
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import srwm_oracle as orc  # noqa: E402


# ---- stand-in extension modules (pybind signatures of the reference) -------------------

def _self_ref_forward(x, W_y, W_q, W_k, w_b, q, k, beta, y_diff, q_diff, k_diff,
                      beta_diff, out):
    f = orc.srwm_forward_explicit(x, W_y, W_q, W_k, w_b)
    # the kernel accumulates into zero-filled outputs and leaves the final state in W_*
    out.add_(f["out"]); q.add_(f["q"]); k.add_(f["k"]); beta.add_(f["beta"])
    y_diff.add_(f["y_diff"]); q_diff.add_(f["q_diff"]); k_diff.add_(f["k_diff"])
    beta_diff.add_(f["beta_diff"])
    W_y.data.copy_(f["W_y"]); W_q.data.copy_(f["W_q"]); W_k.data.copy_(f["W_k"])
    w_b.data.copy_(f["w_b"])


def _self_ref_backward(x, q, k, beta, y_diff, q_diff, k_diff, beta_diff, grad_out,
                       W_y, W_q, W_k, w_b, grad_x, grad_Wy, grad_Wq, grad_Wk, grad_wb):
    r = orc.srwm_backward_explicit(x, q, k, beta, y_diff, q_diff, k_diff, beta_diff,
                                   grad_out, W_y, W_q, W_k, w_b)
    grad_x.add_(r[0]); grad_Wy.add_(r[1]); grad_Wq.add_(r[2]); grad_Wk.add_(r[3])
    grad_wb.add_(r[4])


def _fast_weight_forward(Q, K, V, beta, v_old, v_insert, kv, out):
    f = orc.delta_forward_explicit(Q, K, V, beta, kv)
    out.add_(f["out"]); v_old.add_(f["v_old"]); v_insert.add_(f["v_insert"])
    kv.copy_(f["W"])


def _fast_weight_backward(Q, K, V, beta, v_old, v_insert, grad_out, fw_mem, grad_q,
                          grad_k, grad_v, grad_beta):
    r = orc.delta_backward_explicit(Q, K, V, beta, v_old, v_insert, grad_out, fw_mem)
    grad_q.add_(r[0]); grad_k.add_(r[1]); grad_v.add_(r[2]); grad_beta.add_(r[3])
    fw_mem.copy_(r[4])


def _fake_load(name=None, sources=None, **kw):
    m = types.SimpleNamespace()
    m.self_ref_forward = _self_ref_forward
    m.self_ref_backward = _self_ref_backward
    m.fast_weight_forward = _fast_weight_forward
    m.fast_weight_backward = _fast_weight_backward
    return m


def _run_main(path, class_names):
    """Execute a reference package file as ``__main__`` on the CPU; return (namespace, stdout).

    Edits applied to the source text before ``exec`` (no arithmetic is touched):
      * the Function classes dispatch on ``device.type`` through dicts that only hold the
        key "cuda" (self_ref_v0/__init__.py:36-41); the same callables are registered under
        "cpu" just before the ``__main__`` block;
      * ``device='cuda'`` literals and ``torch.cuda.FloatTensor(..., device='cuda')``
        constructors of the test body are redirected to the CPU;
      * the delta function's ``assert X.device.type is not "cpu"`` is neutralised.
    """
    with open(path) as fh:
        src = fh.read()
    marker = "if __name__ == '__main__':"
    assert marker in src
    add = "".join(
        f"{c}.dot['cpu'] = {c}.dot['cuda']\n"
        f"{c}.dot_backward['cpu'] = {c}.dot_backward['cuda']\n" for c in class_names)
    src = src.replace(marker, add + marker, 1)
    src = re.sub(r"torch\.cuda\.FloatTensor\(\s*([^)]*?),\s*device='cuda'\)",
                 r"torch.FloatTensor(\1)", src, flags=re.S)
    src = src.replace("device='cuda'", "device='cpu'")
    src = src.replace('is not "cpu"', '!= "cuda-required"')
    import torch.utils.cpp_extension as cpp_ext
    real_load = cpp_ext.load
    cpp_ext.load = _fake_load
    ns = {"__name__": "__main__", "__file__": path}
    sink = io.StringIO()
    try:
        with contextlib.redirect_stdout(sink):
            exec(compile(src, path, "exec"), ns)
    finally:
        cpp_ext.load = real_load
    return ns, sink.getvalue()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("MODERN_SRWM_REFERENCE", os.path.join(HERE, "..", "..", "reference")),
                    help="root of the upstream modern-srwm checkout")
    ap.add_argument("--out", default=os.path.join(HERE, "..", "tests", "golden"))
    args = ap.parse_args()
    os.makedirs(args.out, exist_ok=True)
    torch.set_num_threads(max(1, os.cpu_count() or 1))

    # ---- SRWM: shapes 3x5x11x8, seed 111 (self_ref_v0/__init__.py:223,240) ------------
    p = os.path.join(args.reference, "supervised_learning", "self_ref_v0", "__init__.py")
    ns, text = _run_main(p, ["SelfRefv0", "StatefulSelfRefv0"])
    assert "==> All tests pass!" in text, "reference SRWM self test did not complete"
    bsz, n_head, slen, d_head = ns["bsz"], ns["n_head"], ns["slen"], ns["d_head"]
    x_in = torch.softmax(ns["x0"], dim=-1)       # the tensor both paths consume (:289,:294)
    gold = dict(
        shape=(bsz, n_head, slen, d_head),
        x=x_in.detach().clone(),
        W_y=ns["Wy0"].clone(), W_q=ns["Wq0"].clone(), W_k=ns["Wk0"].clone(),
        w_b=ns["wb0"].clone(),
        # reference loop output [L,B,H,E] -> [B,H,L,E]
        out=ns["out2"].detach().permute(1, 2, 0, 3).contiguous(),
        grad_out=torch.ones(bsz, n_head, slen, d_head),     # loss = out.sum()
        grad_x=ns["x2_grad"].detach().contiguous(),
        grad_W_y=ns["W_y2_grad"].detach().clone(), grad_W_q=ns["W_q2_grad"].detach().clone(),
        grad_W_k=ns["W_k2_grad"].detach().clone(), grad_w_b=ns["w_b2_grad"].detach().clone(),
        source="supervised_learning/self_ref_v0/__init__.py __main__ (loop + autograd), seed 111",
    )
    torch.save(gold, os.path.join(args.out, "srwm_main_3x5x11x8.pt"))
    print("SRWM reference self test passed with the oracle as the extension; fixture written")

    # ---- delta: shapes 3x5x11x64 (fast_weight/__init__.py:121-122) ---------------------
    p = os.path.join(args.reference, "supervised_learning", "fast_weight", "__init__.py")
    ns, text = _run_main(p, ["DeltaFastWeight"])
    assert "All tests pass." in text, "reference delta self test did not complete"
    gold = dict(
        shape=(ns["bsz"], ns["n_head"], ns["slen"], ns["d_head"]),
        Q=ns["q0"].clone(), K=ns["k0"].clone(), V=ns["v0"].clone(), beta=ns["beta0"].clone(),
        out=ns["out2"].detach().permute(1, 2, 0, 3).contiguous(),
        grad_out=torch.ones_like(ns["v0"]),
        grad_Q=ns["q2"].grad.clone(), grad_K=ns["k2"].grad.clone(),
        grad_V=ns["v2"].grad.clone(), grad_beta=ns["beta2"].grad.clone(),
        source="supervised_learning/fast_weight/__init__.py __main__ (loop + autograd), seed 111",
    )
    torch.save(gold, os.path.join(args.out, "delta_main_3x5x11x64.pt"))
    print("delta reference self test passed with the oracle as the extension; fixture written")


if __name__ == "__main__":
    main()
