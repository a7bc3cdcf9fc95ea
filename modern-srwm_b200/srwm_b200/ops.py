"""Host-side mirror of the reference's operator interface, on top of the C ABI.

Entry points (same names, positional order, shapes and dtypes as the reference):

    self_ref_v0(x, W_y, W_q, W_k, w_b) -> out
        supervised_learning/self_ref_v0/__init__.py:34-124, alias :216
    stateful_self_ref_v0(x, W_y, W_q, W_k, w_b) -> (out, W_y, W_q, W_k, w_b)
        supervised_learning/self_ref_v0/__init__.py:127-212, alias :217
    fast_weight_delta(Q, K, V, beta, W) -> out
        supervised_learning/fast_weight/__init__.py:26-96, alias :100

Behaviour kept from the reference: the forward leaves the FINAL fast-weight state in the
caller's ``W_*`` / ``W`` tensors (callers derive the carried state from that), the delta
backward puts ``W_0`` back, the SRWM backward leaves ``W_L``; gradients are returned per
sample; the delta function returns ``None`` for the state.  Differences, all deliberate:
outputs are written with plain stores (no zero-filled buffers needed), the whole sequence
is one launch (no limit on L), head dims 32/64 are correct in the backward, the stateful
backward returns the true dL/dW_0, activations may be bfloat16 (state stays fp32), and
the call runs on the tensors' device and torch's current stream.

There is no CPU implementation: tensors must live on a CUDA device and the prebuilt
library must be present, otherwise the call raises.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _lib as L

_OPS = {"srwm_fwd": L.OP_SRWM_FWD, "srwm_bwd": L.OP_SRWM_BWD,
        "delta_fwd": L.OP_DELTA_FWD, "delta_bwd": L.OP_DELTA_BWD}
_variants = {}   # (op_name, E) -> variant id


def set_variant(op, E, variant):
    """Select a compiled kernel configuration (tuning aid; 0 = default)."""
    assert op in _OPS
    _variants[(op, int(E))] = int(variant)


def _load_env_variants():
    # SRWM_B200_VARIANTS="srwm_bwd:64=1,delta_fwd:64=2"
    spec = os.environ.get("SRWM_B200_VARIANTS", "")
    for item in filter(None, spec.split(",")):
        k, v = item.split("=")
        op, e = k.split(":")
        set_variant(op.strip(), int(e), int(v))


_load_env_variants()


def _variant(op, E):
    return _variants.get((op, E), 0)


# ---------------------------------------------------------------------------------------
# tensor -> ABI descriptors
# ---------------------------------------------------------------------------------------

def _io_dtype(t):
    if t.dtype == torch.float32:
        return L.F32
    if t.dtype == torch.bfloat16:
        return L.BF16
    raise TypeError(f"activations must be float32 or bfloat16, got {t.dtype}")


def _require_cuda(*ts):
    for t in ts:
        if t.device.type != "cuda":
            raise RuntimeError(
                "srwm_b200 operators run on CUDA tensors only (no CPU implementation); "
                f"got a tensor on {t.device}")


def _seq_ok(t):
    """innermost contiguous and every row 16-byte aligned (strides of size-1 dims ignored)."""
    es = t.element_size()
    sh, st = t.shape, t.stride()
    if sh[3] > 1 and st[3] != 1:
        return False
    if t.data_ptr() % 16:
        return False
    for d in range(3):
        if sh[d] > 1 and (st[d] * es) % 16:
            return False
    return True


def _seq(t):
    """Return a tensor usable as an ABI sequence view (copying only when it must)."""
    return t if _seq_ok(t) else t.contiguous()


def _seq_desc(t):
    sh, st = t.shape, t.stride()
    return L.Seq(t.data_ptr(), st[0] if sh[0] > 1 else 0, st[1] if sh[1] > 1 else 0, st[2] if sh[2] > 1 else 0)


_narrow_desc = _seq_desc      # [N,H,L,1] tensors (delta beta): any strides


def _state_ok(t):
    if t.dtype is not torch.float32 or t.data_ptr() % 16:
        return False
    sh, st = t.shape, t.stride()
    if st[3] != 1 or st[2] != sh[3]:
        return False
    for d in range(2):
        if sh[d] > 1 and (st[d] * 4) % 16:
            return False
    return True


def _state_desc(t):
    sh, st = t.shape, t.stride()
    return L.State(t.data_ptr(), st[0] if sh[0] > 1 else 0, st[1] if sh[1] > 1 else 0)


def _like(t, last=None):
    """Uninitialised tensor with the shape of ``t`` (optionally another last dimension) laid
    out in memory like ``t``.  The layers hand in permuted views of ``[L, B, H*d]``
    activations (supervised_learning/layer.py:161-165) and turn the result back with
    ``transpose(1, 2).reshape(B, L, H*d)`` (:184-186); when the output follows the input's
    memory order that reshape is a view instead of a full copy, and the same holds for the
    gradients on the way back."""
    if last is None or last == t.size(-1):
        return torch.empty_like(t)      # preserve_format keeps the strides of a dense permuted view
    shape = tuple(t.shape[:-1]) + (last,)
    order = sorted(range(3), key=lambda d: (-t.stride(d), d))      # outer-to-inner memory order
    strides = [0, 0, 0, 1]
    run = last
    for d in reversed(order):
        strides[d] = run
        run *= shape[d]
    return torch.empty_strided(shape, strides, device=t.device, dtype=t.dtype)


_NULL_SEQ = L.Seq(None, 0, 0, 0)
_NULL_STATE = L.State(None, 0, 0)


def _stream(t):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


class _StateIO:
    """In/out state tensors: the kernel works on a dense fp32 tensor; if the caller's
    tensor is not, work on a dense copy and copy the result back (the in-place side
    effect is part of the interface)."""

    def __init__(self, *tensors):
        self.orig = tensors
        self.work = [t if _state_ok(t) else t.detach().to(torch.float32).contiguous() for t in tensors]

    def writeback(self):
        for o, w in zip(self.orig, self.work):
            if o is not w:
                o.detach().copy_(w)


# ---------------------------------------------------------------------------------------
# raw (non-autograd) calls
# ---------------------------------------------------------------------------------------

def srwm_forward(x, W_y, W_q, W_k, w_b, save=True, variant=None):
    """Run the SRWM forward kernel.  Mutates W_* to the final state.
    Returns (out, saved) with saved = (q, k, beta, y_diff, q_diff, k_diff, beta_diff) or None."""
    _require_cuda(x, W_y, W_q, W_k, w_b)
    N, H, Ln, E = x.shape
    assert W_y.shape == (N, H, E, E), "Reshape/unsqueeze if needed."
    assert W_q.shape == (N, H, E, E), "Reshape/unsqueeze if needed."
    assert W_k.shape == (N, H, E, E), "Reshape/unsqueeze if needed."
    assert w_b.shape == (N, H, E, 4), "Reshape/unsqueeze if needed."
    dt = _io_dtype(x)
    xs = _seq(x.detach())
    st = _StateIO(W_y, W_q, W_k, w_b)
    dev = x.device
    out = _like(xs)
    a = L.SrwmFwdArgs()
    a.N, a.H, a.L, a.E = N, H, Ln, E
    a.io_dtype = dt
    a.flags = 0 if save else L.FLAG_NO_SAVE
    a.variant = _variant("srwm_fwd", E) if variant is None else variant
    a.x = _seq_desc(xs)
    a.W_y, a.W_q, a.W_k, a.w_b = (_state_desc(t) for t in st.work)
    a.out = _seq_desc(out)
    saved = None
    if save:
        # two allocations for the seven saved tensors (they live and die together)
        q, k, yd, qd, kd = torch.empty((5, N, H, Ln, E), device=dev, dtype=torch.float32).unbind(0)
        beta, bd = torch.empty((2, N, H, Ln, 4), device=dev, dtype=torch.float32).unbind(0)
        saved = (q, k, beta, yd, qd, kd, bd)
        a.q, a.k, a.beta = _seq_desc(q), _seq_desc(k), _seq_desc(beta)
        a.y_diff, a.q_diff, a.k_diff, a.beta_diff = (_seq_desc(t) for t in (yd, qd, kd, bd))
    else:
        a.q = a.k = a.beta = a.y_diff = a.q_diff = a.k_diff = a.beta_diff = _NULL_SEQ
    with torch.cuda.device(dev):
        L.check(L.load().srwm_b200_srwm_forward(C.byref(a), _stream(x)), "srwm_forward")
    st.writeback()
    return out, saved


def srwm_backward(x, saved, grad_out, W_y, W_q, W_k, w_b, grad_state=None, restore_state=False,
                  variant=None):
    """Run the SRWM backward kernel.  W_* must hold the final state of the forward.
    grad_state: optional (gW_y, gW_q, gW_k, gw_b) = dL/d(final state); never modified.
    Returns (grad_x, grad_W_y, grad_W_q, grad_W_k, grad_w_b) (dL/dW_0, per sample)."""
    _require_cuda(x, grad_out, W_y)
    N, H, Ln, E = x.shape
    dt = _io_dtype(x)
    q, k, beta, yd, qd, kd, bd = saved
    xs = _seq(x.detach())
    go = grad_out.detach()
    if go.dtype != x.dtype:
        go = go.to(x.dtype)
    go = _seq(go)
    st = _StateIO(W_y, W_q, W_k, w_b)
    dev = x.device
    grad_x = _like(xs)
    flags = 0
    if grad_state is not None and any(g is not None for g in grad_state):
        shapes = [(N, H, E, E)] * 3 + [(N, H, E, 4)]
        gW = [(g.detach().to(torch.float32).contiguous().clone() if g is not None
               else torch.zeros(s, device=dev, dtype=torch.float32))
              for g, s in zip(grad_state, shapes)]
        flags |= L.FLAG_STATE_GRAD_IN
    else:
        gW = [torch.empty((N, H, E, E), device=dev, dtype=torch.float32) for _ in range(3)]
        gW.append(torch.empty((N, H, E, 4), device=dev, dtype=torch.float32))
    if restore_state:
        flags |= L.FLAG_RESTORE_STATE
    a = L.SrwmBwdArgs()
    a.N, a.H, a.L, a.E = N, H, Ln, E
    a.io_dtype = dt
    a.flags = flags
    a.variant = _variant("srwm_bwd", E) if variant is None else variant
    a.x = _seq_desc(xs)
    a.q, a.k, a.beta = _seq_desc(q), _seq_desc(k), _seq_desc(beta)
    a.y_diff, a.q_diff, a.k_diff, a.beta_diff = (_seq_desc(t) for t in (yd, qd, kd, bd))
    a.grad_out = _seq_desc(go)
    a.W_y, a.W_q, a.W_k, a.w_b = (_state_desc(t) for t in st.work)
    a.grad_x = _seq_desc(grad_x)
    a.grad_W_y, a.grad_W_q, a.grad_W_k, a.grad_w_b = (_state_desc(t) for t in gW)
    with torch.cuda.device(dev):
        L.check(L.load().srwm_b200_srwm_backward(C.byref(a), _stream(x)), "srwm_backward")
    if restore_state:
        st.writeback()
    return (grad_x, *gW)


def delta_forward(Q, K, V, beta, W, save=True, variant=None):
    """Run the delta-rule forward kernel.  Mutates W to the final state.
    Returns (out, saved) with saved = (v_old, v_insert) or None."""
    _require_cuda(Q, K, V, beta, W)
    N, H, Ln, E = Q.shape
    M = V.shape[-1]
    assert K.shape == (N, H, Ln, E) and V.shape == (N, H, Ln, M)
    assert beta.shape == (N, H, Ln, 1) and W.shape == (N, H, E, M)
    dt = _io_dtype(Q)
    Qs, Ks, Vs = (_seq(t.detach().to(Q.dtype)) for t in (Q, K, V))
    bs = beta.detach().to(Q.dtype)
    st = _StateIO(W)
    dev = Q.device
    out = _like(Qs, M)
    a = L.DeltaFwdArgs()
    a.N, a.H, a.L, a.E, a.M = N, H, Ln, E, M
    a.io_dtype = dt
    a.flags = 0 if save else L.FLAG_NO_SAVE
    a.variant = _variant("delta_fwd", E) if variant is None else variant
    a.Q, a.K, a.V, a.beta = _seq_desc(Qs), _seq_desc(Ks), _seq_desc(Vs), _narrow_desc(bs)
    a.W = _state_desc(st.work[0])
    a.out = _seq_desc(out)
    saved = None
    if save:
        v_old = torch.empty((N, H, Ln, M), device=dev, dtype=torch.float32)
        v_ins = torch.empty((N, H, Ln, M), device=dev, dtype=torch.float32)
        saved = (v_old, v_ins)
        a.v_old, a.v_insert = _seq_desc(v_old), _seq_desc(v_ins)
    else:
        a.v_old = a.v_insert = _NULL_SEQ
    with torch.cuda.device(dev):
        L.check(L.load().srwm_b200_delta_forward(C.byref(a), _stream(Q)), "delta_forward")
    st.writeback()
    return out, saved


def delta_backward(Q, K, V, beta, saved, grad_out, W, want_grad_W0=False, variant=None):
    """Run the delta-rule backward kernel.  W holds W_L on entry, W_0 on return.
    Returns (grad_Q, grad_K, grad_V, grad_beta, grad_W0 or None)."""
    _require_cuda(Q, grad_out, W)
    N, H, Ln, E = Q.shape
    M = V.shape[-1]
    dt = _io_dtype(Q)
    v_old, v_ins = saved
    Qs, Ks, Vs = (_seq(t.detach().to(Q.dtype)) for t in (Q, K, V))
    bs = beta.detach().to(Q.dtype)
    go = _seq(grad_out.detach().to(Q.dtype))
    st = _StateIO(W)
    dev = Q.device
    gQ = _like(Qs)
    gK = _like(Ks)
    gV = _like(Qs, M)
    gB = torch.empty((N, H, Ln, 1), device=dev, dtype=Q.dtype)
    gW0 = torch.empty((N, H, E, M), device=dev, dtype=torch.float32) if want_grad_W0 else None
    a = L.DeltaBwdArgs()
    a.N, a.H, a.L, a.E, a.M = N, H, Ln, E, M
    a.io_dtype = dt
    a.flags = 0
    a.variant = _variant("delta_bwd", E) if variant is None else variant
    a.Q, a.K, a.V, a.beta = _seq_desc(Qs), _seq_desc(Ks), _seq_desc(Vs), _narrow_desc(bs)
    a.v_old, a.v_insert = _seq_desc(v_old), _seq_desc(v_ins)
    a.grad_out = _seq_desc(go)
    a.W = _state_desc(st.work[0])
    a.grad_Q, a.grad_K, a.grad_V = _seq_desc(gQ), _seq_desc(gK), _seq_desc(gV)
    a.grad_beta = _narrow_desc(gB)
    a.grad_W0 = _state_desc(gW0) if want_grad_W0 else _NULL_STATE
    with torch.cuda.device(dev):
        L.check(L.load().srwm_b200_delta_backward(C.byref(a), _stream(Q)), "delta_backward")
    st.writeback()
    return gQ, gK, gV, gB, gW0


def reduce_batch(src, dst=None, accumulate=False):
    """Sum per-sample state gradients [N, ...] over the batch into dst [...] (fp32)."""
    _require_cuda(src)
    assert src.dtype == torch.float32
    src = src.contiguous()
    N = src.shape[0]
    count = src[0].numel() if N > 0 else 0
    if dst is None:
        dst = torch.empty(src.shape[1:], device=src.device, dtype=torch.float32)
        accumulate = False
    assert dst.is_contiguous() and dst.numel() == count and dst.dtype == torch.float32
    with torch.cuda.device(src.device):
        L.check(L.load().srwm_b200_reduce_batch(src.data_ptr(), count, N, count, dst.data_ptr(),
                                                1 if accumulate else 0, _stream(src)), "reduce_batch")
    return dst


# ---------------------------------------------------------------------------------------
# autograd boundary (reference names)
# ---------------------------------------------------------------------------------------

class SelfRefv0(torch.autograd.Function):
    """supervised_learning/self_ref_v0/__init__.py:34-124."""

    @staticmethod
    def forward(ctx, x, W_y, W_q, W_k, w_b):
        need = any(ctx.needs_input_grad)
        out, saved = srwm_forward(x, W_y, W_q, W_k, w_b, save=need)
        if need:
            ctx.save_for_backward(x, *saved, W_y, W_q, W_k, w_b)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x, q, k, beta, yd, qd, kd, bd, W_y, W_q, W_k, w_b = ctx.saved_tensors
        return srwm_backward(x, (q, k, beta, yd, qd, kd, bd), grad_out, W_y, W_q, W_k, w_b)


class StatefulSelfRefv0(torch.autograd.Function):
    """supervised_learning/self_ref_v0/__init__.py:127-212: also returns the (mutated)
    state tensors and accepts gradients flowing into them."""

    @staticmethod
    def forward(ctx, x, W_y, W_q, W_k, w_b):
        need = any(ctx.needs_input_grad)
        out, saved = srwm_forward(x, W_y, W_q, W_k, w_b, save=need)
        if need:
            ctx.save_for_backward(x, *saved, W_y, W_q, W_k, w_b)
        return out, W_y, W_q, W_k, w_b

    @staticmethod
    def backward(ctx, grad_out, grad_W_y, grad_W_q, grad_W_k, grad_w_b):
        x, q, k, beta, yd, qd, kd, bd, W_y, W_q, W_k, w_b = ctx.saved_tensors
        if grad_out is None:
            grad_out = torch.zeros_like(x)
        return srwm_backward(x, (q, k, beta, yd, qd, kd, bd), grad_out, W_y, W_q, W_k, w_b,
                             grad_state=(grad_W_y, grad_W_q, grad_W_k, grad_w_b))


class DeltaFastWeight(torch.autograd.Function):
    """Fast weight using the delta update rule
    (supervised_learning/fast_weight/__init__.py:26-96)."""

    @staticmethod
    def forward(ctx, Q, K, V, beta, W):
        need = any(ctx.needs_input_grad[:4])
        out, saved = delta_forward(Q, K, V, beta, W, save=need)
        if need:
            ctx.save_for_backward(Q, K, V, beta, *saved, W)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        Q, K, V, beta, v_old, v_ins, W = ctx.saved_tensors
        gQ, gK, gV, gB, _ = delta_backward(Q, K, V, beta, (v_old, v_ins), grad_out, W)
        return gQ.to(Q.dtype), gK.to(K.dtype), gV.to(V.dtype), gB.to(beta.dtype), None


def _no_grad_needed(*ts):
    return not (torch.is_grad_enabled() and any(t.requires_grad for t in ts))


def self_ref_v0(x, W_y, W_q, W_k, w_b):
    """``SelfRefv0.apply`` (supervised_learning/self_ref_v0/__init__.py:216); when nothing needs a
    gradient (the actors' single-step calls) the autograd machinery is skipped."""
    if _no_grad_needed(x, W_y, W_q, W_k, w_b):
        return srwm_forward(x, W_y, W_q, W_k, w_b, save=False)[0]
    return SelfRefv0.apply(x, W_y, W_q, W_k, w_b)


def stateful_self_ref_v0(x, W_y, W_q, W_k, w_b):
    """``StatefulSelfRefv0.apply`` (supervised_learning/self_ref_v0/__init__.py:217)."""
    if _no_grad_needed(x, W_y, W_q, W_k, w_b):
        return (srwm_forward(x, W_y, W_q, W_k, w_b, save=False)[0], W_y, W_q, W_k, w_b)
    return StatefulSelfRefv0.apply(x, W_y, W_q, W_k, w_b)


def fast_weight_delta(Q, K, V, beta, W):
    """``DeltaFastWeight.apply`` (supervised_learning/fast_weight/__init__.py:100)."""
    if _no_grad_needed(Q, K, V, beta):
        return delta_forward(Q, K, V, beta, W, save=False)[0]
    return DeltaFastWeight.apply(Q, K, V, beta, W)
