"""The allocation-free variant of the layer-level backward with fused batch reduction
(``srwm_b200_srwm_layer_backward_reduced_static``), called through the C ABI.

That entry point exists for hosts that have no way to obtain a scratch block: code that runs on
buffers handed to it by an application whose device memory is owned by someone else's pool, and
loops that must not pay for (or be stalled by) a ``cudaMalloc`` in the call path.  It keeps its
working memory in an array inside the library instead of taking it from the caller.

Checked here: on the same inputs it returns what the caller-scratch entry point returns (same
kernel, same fixed summation order -- the comparison still uses the tolerance of the other
reduction tests), on two calls in a row with different upstream gradients, so that a call sees
whatever the previous one left in the shared array; and a size beyond the array is refused.
This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-5      # as in test_fused_batch_reduction_matches_the_separate_one


def _rel_max(a, b):
    a, b = a.double(), b.double()
    return float((a - b).abs().max() / (b.abs().max() + 1e-300))


def _backward(lib_fn, x, saved, go, base, shift_out, scratch):
    """One call of a reduced layer backward through ctypes; returns (grad_x, per-sample grads, sums)."""
    from srwm_b200 import _lib as L
    from srwm_b200.ops import _seq_desc, _state_desc, _stream
    N, H, Ln, E = x.shape
    d = x.device
    q, k, beta, yd, qd, kd, bd = saved
    grad_x = torch.empty_like(x)
    gW = [torch.empty(N, H, E, w, device=d) for w in (E, E, E, 4)]
    sums = [torch.full((1, H, E, w), float("nan"), device=d) for w in (E, E, E, 4)]
    a = L.SrwmBwdArgs()
    a.N, a.H, a.L, a.E = N, H, Ln, E
    a.io_dtype, a.flags, a.variant = L.F32, L.FLAG_INPUT_SOFTMAX, 0
    a.x = _seq_desc(x)
    a.q, a.k, a.beta = _seq_desc(q), _seq_desc(k), _seq_desc(beta)
    a.y_diff, a.q_diff, a.k_diff, a.beta_diff = (_seq_desc(t) for t in (yd, qd, kd, bd))
    a.grad_out = _seq_desc(go)
    a.W_y, a.W_q, a.W_k, a.w_b = (_state_desc(t) for t in shift_out)
    a.grad_x = _seq_desc(grad_x)
    a.grad_W_y, a.grad_W_q, a.grad_W_k, a.grad_w_b = (_state_desc(t) for t in gW)
    e = L.SrwmExt()
    e.base_W_y, e.base_W_q, e.base_W_k, e.base_w_b = (_state_desc(t) for t in base)
    r = L.SrwmReduce()
    r.grad_base_W_y, r.grad_base_W_q, r.grad_base_W_k = (L.State(t.data_ptr(), 0, E * E) for t in sums[:3])
    r.grad_base_w_b = L.State(sums[3].data_ptr(), 0, E * 4)
    r.accumulate = 0
    if scratch is not None:
        r.scratch, r.scratch_bytes = scratch.data_ptr(), scratch.numel()
    L.check(lib_fn(C.byref(a), C.byref(e), C.byref(r), _stream(x)), "reduced layer backward")
    torch.cuda.synchronize()
    return grad_x, gW, sums


@pytest.mark.parametrize("N,E", [(40, 64), (130, 32)])      # one group of samples; five groups (two levels)
def test_static_scratch_variant_matches_caller_scratch_variant(N, E):
    from srwm_b200 import _lib as L
    from srwm_b200 import layer_ops as lo
    lib = L.load()
    d = torch.device("cuda", 0)
    torch.cuda.set_device(d)
    H, Ln = 3, 24
    g = torch.Generator().manual_seed(7 + N)
    x = torch.randn(N, H, Ln, E, generator=g).to(d)
    std = E ** -0.5
    base = [(torch.randn(1, H, E, w, generator=g) * std).to(d) for w in (E, E, E, 4)]
    _, shift_out, saved = lo.srwm_layer_forward(x, base, None, None, True)
    need = int(lib.srwm_b200_srwm_reduce_scratch_bytes(N, H, E))
    assert 0 < need <= L.STATIC_SCRATCH_BYTES
    scratch = torch.zeros(need, dtype=torch.uint8, device=d)
    for call in range(2):                                    # the second call finds the first one's leftovers
        go = torch.randn(N, H, Ln, E, generator=g).to(d)
        ref = _backward(lib.srwm_b200_srwm_layer_backward_reduced, x, saved, go, base, shift_out, scratch)
        got = _backward(lib.srwm_b200_srwm_layer_backward_reduced_static, x, saved, go, base, shift_out, None)
        assert _rel_max(got[0], ref[0]) < TOL, call
        for a, b in zip(got[1], ref[1]):
            assert _rel_max(a, b) < TOL, call
        for a, b in zip(got[2], ref[2]):
            assert not bool(torch.isnan(a).any())
            assert _rel_max(a, b) < TOL, call
        want = [t.double().sum(0, keepdim=True) for t in ref[1]]
        for a, b in zip(got[2], want):
            assert _rel_max(a, b) < TOL, call


def test_static_scratch_variant_refuses_what_does_not_fit():
    from srwm_b200 import _lib as L
    lib = L.load()
    a = L.SrwmBwdArgs()
    a.N, a.H, a.L, a.E = 1024, 16, 8, 64        # needs about 26 MB of group partials
    r = L.SrwmReduce()
    assert int(lib.srwm_b200_srwm_reduce_scratch_bytes(1024, 16, 64)) > L.STATIC_SCRATCH_BYTES
    assert lib.srwm_b200_srwm_layer_backward_reduced_static(C.byref(a), None, C.byref(r), None) == L.ERR_TOO_LARGE
    assert b"exceeds" in lib.srwm_b200_strerror(L.ERR_TOO_LARGE)
    assert lib.srwm_b200_srwm_layer_backward_reduced_static(None, None, C.byref(r), None) == L.ERR_NULL
