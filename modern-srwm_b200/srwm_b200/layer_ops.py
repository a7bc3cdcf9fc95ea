"""Layer-level SRWM calls: what the reference's layers do around ``self_ref_v0``, taken into
the kernels (C entry points ``srwm_b200_srwm_layer_forward`` / ``_layer_backward`` /
``srwm_b200_srwm_backward_detached``).

    srwm_layer(x, W_y, W_q, W_k, w_b, shift=None, done=None, input_softmax=True,
               detach_state=False) -> (out, (shift_W_y, shift_W_q, shift_W_k, shift_w_b))

replaces, in one call,

* the input softmax (supervised_learning/layer.py:162-163,
  reinforcement_learning/torchbeast/layer.py:383),
* ``W.repeat(bsz, 1, 1, 1)`` of the four slow weights and ``shift + repeat``
  (supervised_learning/layer.py:166-177, torchbeast/layer.py:392-395): the slow weights stay
  ``[1, H, d, .]`` and are read with a batch stride of zero,
* the operator itself,
* ``W_bc - W.repeat(bsz, 1, 1, 1)`` for the new carried state (layer.py:200-204 / :412-415),
* with ``done``: the learner's one-step-at-a-time loop with ``state * notdone`` before every
  step (reinforcement_learning/torchbeast_procgen/model.py:1180-1197).

Gradients.  ``detach_state=False``: backpropagation through time over the whole call; the
slow weights receive the batch sum of the per-sample dL/dW_0 (minus the incoming dL/dshift),
the initial shift the per-sample dL/dW_0.  ``detach_state=True``: the reference learner's
gradient, i.e. every step sees a detached state (torchbeast/layer.py:412-421): only W_y and x
receive gradient, W_q / W_k / w_b get zeros; required when ``done`` is given.

    delta_layer(qkvb, W, norm_eps=0.0, zero_init=False) -> out

is the same for the delta-rule layers (``FastFFlayer``, supervised_learning/layer.py:49-108 and
reinforcement_learning/torchbeast/layer.py:127-189): it reads the raw ``slow_net`` rows
``[q | k | v | b]`` in place -- no split copies -- applies ``elu + 1``, the sum normalisation
(``norm_eps`` = 0 in the supervised layer, 1e-5 in the agents') and the sigmoid inside the
kernels, and returns the gradient of the raw rows in the same packed layout.

CUDA tensors only; there is no CPU implementation.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L
from .ops import (_NULL_SEQ, _NULL_STATE, _io_dtype, _like, _require_cuda, _seq, _seq_desc, _state_desc,
                  _state_ok, _stream, reduce_batch)


def _dense_state(t):
    return t if _state_ok(t) else t.detach().to(torch.float32).contiguous()


def _ext(base, shift=None, done=None):
    e = L.SrwmExt()
    e.base_W_y, e.base_W_q, e.base_W_k, e.base_w_b = (_state_desc(t) for t in base)
    if shift is not None:
        e.shift_W_y, e.shift_W_q, e.shift_W_k, e.shift_w_b = (_state_desc(t) for t in shift)
    else:
        e.shift_W_y = e.shift_W_q = e.shift_W_k = e.shift_w_b = _NULL_STATE
    if done is not None:
        e.done = done.data_ptr()
        e.done_stride_n, e.done_stride_l = done.stride(0), done.stride(1)
    else:
        e.done = None
        e.done_stride_n = e.done_stride_l = 0
    return e


def _done_bytes(done, N, Ln):
    """[N, L] reset flags as a uint8 tensor (any strides; a [T, B] learner mask is passed as its
    transposed view)."""
    if done is None:
        return None
    assert done.shape == (N, Ln), "done must be [N, L]"
    if done.dtype == torch.bool:
        return done.view(torch.uint8)
    if done.dtype == torch.uint8:
        return done
    return (done != 0).view(torch.uint8)


def srwm_layer_forward(x, base, shift=None, done=None, input_softmax=True, save=True, inplace_state=False,
                       variant=0):
    """Forward.  x [N,H,L,E] (raw activations with ``input_softmax``), base = 4 slow-weight
    tensors [1,H,E,.] (or per sample [N,H,E,.]), shift = optional 4 tensors [N,H,E,.], done =
    optional [N,L].  Returns (out, shift_out (4 new tensors), saved or None).
    ``inplace_state``: write the new shift over the given one (inference only: every thread
    overwrites exactly the state elements it read at the start, but a backward would no longer
    find its initial shift).  ``variant``: kernel configuration id (0 = the library chooses)."""
    _require_cuda(x, *base)
    N, H, Ln, E = x.shape
    shapes = [(E, E)] * 3 + [(E, 4)]
    for b, s in zip(base, shapes):
        assert b.dim() == 4 and b.shape[0] in (1, N) and b.shape[1] == H and tuple(b.shape[2:]) == s, \
            "slow weights must be [1 or N, H, E, E] / [1 or N, H, E, 4]"
    dt = _io_dtype(x)
    xs = _seq(x.detach())
    dev = x.device
    base = [_dense_state(b.detach()) for b in base]
    if shift is not None:
        for sft, s in zip(shift, shapes):
            assert tuple(sft.shape) == (N, H) + s, "shift must be [N, H, E, E] / [N, H, E, 4]"
        shift = [_dense_state(s.detach()) for s in shift]
    done_b = _done_bytes(done, N, Ln)
    out = _like(xs)
    if inplace_state:
        assert shift is not None and not save, "in-place state update is for inference calls with a carried state"
        shift_out = shift
    else:
        shift_out = [torch.empty((N, H) + s, device=dev, dtype=torch.float32) for s in shapes]
    a = L.SrwmFwdArgs()
    a.N, a.H, a.L, a.E = N, H, Ln, E
    a.io_dtype = dt
    a.flags = (0 if save else L.FLAG_NO_SAVE) | (L.FLAG_INPUT_SOFTMAX if input_softmax else 0)
    a.variant = variant
    a.x = _seq_desc(xs)
    a.W_y, a.W_q, a.W_k, a.w_b = (_state_desc(t) for t in shift_out)
    a.out = _seq_desc(out)
    saved = None
    if save:
        q, k, yd, qd, kd = torch.empty((5, N, H, Ln, E), device=dev, dtype=torch.float32).unbind(0)
        beta, bd = torch.empty((2, N, H, Ln, 4), device=dev, dtype=torch.float32).unbind(0)
        saved = (q, k, beta, yd, qd, kd, bd)
        a.q, a.k, a.beta = _seq_desc(q), _seq_desc(k), _seq_desc(beta)
        a.y_diff, a.q_diff, a.k_diff, a.beta_diff = (_seq_desc(t) for t in (yd, qd, kd, bd))
    else:
        a.q = a.k = a.beta = a.y_diff = a.q_diff = a.k_diff = a.beta_diff = _NULL_SEQ
    if Ln == 0:      # nothing to run: the state is carried through unchanged
        if not inplace_state:
            for so, si in zip(shift_out, shift if shift is not None else [None] * 4):
                so.zero_() if si is None else so.copy_(si)
        return out, shift_out, saved
    e = _ext(base, shift, done_b)
    with torch.cuda.device(dev):
        L.check(L.load().srwm_b200_srwm_layer_forward(C.byref(a), C.byref(e), _stream(x)), "srwm_layer_forward")
    return out, shift_out, saved


_reduce_scratch = {}     # (device index, stream) -> scratch tensor of the fused batch reduction


def _scratch_for(dev, nbytes):
    """Working memory of the fused batch reduction, kept per (device, stream): calls on one stream
    are ordered, so they can share it; calls on different streams may overlap and must not."""
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    t = _reduce_scratch.get(key)
    if t is None or t.numel() < nbytes:
        t = torch.zeros(max(nbytes, 1024), dtype=torch.uint8, device=dev)
        _reduce_scratch[key] = t
    return t


def srwm_layer_backward(x, saved, grad_out, base, shift_out, grad_shift_out=None, input_softmax=True,
                        reduce_into=None, accumulate=False):
    """Backpropagation through time for ``srwm_layer_forward`` (no ``done``).  shift_out: the
    forward's final shift (left unchanged).  Returns (grad_x, gW_y, gW_q, gW_k, gw_b) with the
    state gradients per sample (dL/dW_0).
    ``reduce_into``: four dense fp32 tensors ``[1,H,E,.]`` (e.g. views into a flat all-reduce bucket)
    that receive the batch sums of those gradients, formed inside the backward kernel
    (``accumulate``: added to their contents)."""
    _require_cuda(x, grad_out)
    N, H, Ln, E = x.shape
    dt = _io_dtype(x)
    q, k, beta, yd, qd, kd, bd = saved
    xs = _seq(x.detach())
    go = grad_out.detach()
    if go.dtype != x.dtype:
        go = go.to(x.dtype)
    go = _seq(go)
    dev = x.device
    base = [_dense_state(b.detach()) for b in base]
    grad_x = _like(xs)
    shapes = [(N, H, E, E)] * 3 + [(N, H, E, 4)]
    flags = L.FLAG_INPUT_SOFTMAX if input_softmax else 0
    if grad_shift_out is not None and any(g is not None for g in grad_shift_out):
        gW = [(g.detach().to(torch.float32).contiguous().clone() if g is not None
               else torch.zeros(s, device=dev, dtype=torch.float32))
              for g, s in zip(grad_shift_out, shapes)]
        flags |= L.FLAG_STATE_GRAD_IN
    else:
        gW = [torch.empty(s, device=dev, dtype=torch.float32) for s in shapes]
    a = L.SrwmBwdArgs()
    a.N, a.H, a.L, a.E = N, H, Ln, E
    a.io_dtype = dt
    a.flags = flags
    a.variant = 0
    a.x = _seq_desc(xs)
    a.q, a.k, a.beta = _seq_desc(q), _seq_desc(k), _seq_desc(beta)
    a.y_diff, a.q_diff, a.k_diff, a.beta_diff = (_seq_desc(t) for t in (yd, qd, kd, bd))
    a.grad_out = _seq_desc(go)
    a.W_y, a.W_q, a.W_k, a.w_b = (_state_desc(t) for t in shift_out)
    a.grad_x = _seq_desc(grad_x)
    a.grad_W_y, a.grad_W_q, a.grad_W_k, a.grad_w_b = (_state_desc(t) for t in gW)
    e = _ext(base)
    if reduce_into is None:
        with torch.cuda.device(dev):
            L.check(L.load().srwm_b200_srwm_layer_backward(C.byref(a), C.byref(e), _stream(x)), "srwm_layer_backward")
        return (grad_x, *gW)
    for t, w in zip(reduce_into, (E, E, E, 4)):
        assert t.dtype == torch.float32 and t.is_contiguous() and t.numel() == H * E * w, \
            "reduce_into: four dense fp32 tensors [1,H,E,E] x3, [1,H,E,4]"
    r = L.SrwmReduce()
    r.grad_base_W_y, r.grad_base_W_q, r.grad_base_W_k = (L.State(t.data_ptr(), 0, E * E) for t in reduce_into[:3])
    r.grad_base_w_b = L.State(reduce_into[3].data_ptr(), 0, E * 4)
    r.accumulate = 1 if accumulate else 0
    with torch.cuda.device(dev):
        lib = L.load()
        nbytes = int(lib.srwm_b200_srwm_reduce_scratch_bytes(N, H, E))
        scratch = _scratch_for(dev, nbytes)
        r.scratch, r.scratch_bytes = scratch.data_ptr(), scratch.numel()
        L.check(lib.srwm_b200_srwm_layer_backward_reduced(C.byref(a), C.byref(e), C.byref(r), _stream(x)),
                "srwm_layer_backward_reduced")
    return (grad_x, *gW)


def srwm_backward_detached(x, saved, grad_out, base_W_y, shift_W_y=None, done=None, input_softmax=True):
    """Backward with the state detached at every step.  saved: the forward's saved tuple (k,
    beta, y_diff are used).  Returns (grad_x, grad_W_y per sample [N,H,E,E])."""
    _require_cuda(x, grad_out, base_W_y)
    N, H, Ln, E = x.shape
    dt = _io_dtype(x)
    _, k, beta, yd, _, _, _ = saved
    xs = _seq(x.detach())
    go = grad_out.detach()
    if go.dtype != x.dtype:
        go = go.to(x.dtype)
    go = _seq(go)
    dev = x.device
    base_W_y = _dense_state(base_W_y.detach())
    if shift_W_y is not None:
        shift_W_y = _dense_state(shift_W_y.detach())
    done_b = _done_bytes(done, N, Ln)
    grad_x = _like(xs)
    gWy = torch.empty((N, H, E, E), device=dev, dtype=torch.float32)
    a = L.SrwmBwdDetArgs()
    a.N, a.H, a.L, a.E = N, H, Ln, E
    a.io_dtype = dt
    a.flags = L.FLAG_INPUT_SOFTMAX if input_softmax else 0
    a.variant = 0
    a.x = _seq_desc(xs)
    a.k, a.beta, a.y_diff = _seq_desc(k), _seq_desc(beta), _seq_desc(yd)
    a.grad_out = _seq_desc(go)
    a.base_W_y = _state_desc(base_W_y)
    a.shift_W_y = _state_desc(shift_W_y) if shift_W_y is not None else _NULL_STATE
    if done_b is not None:
        a.done = done_b.data_ptr()
        a.done_stride_n, a.done_stride_l = done_b.stride(0), done_b.stride(1)
    else:
        a.done = None
        a.done_stride_n = a.done_stride_l = 0
    a.grad_x = _seq_desc(grad_x)
    a.grad_W_y = _state_desc(gWy)
    with torch.cuda.device(dev):
        L.check(L.load().srwm_b200_srwm_backward_detached(C.byref(a), _stream(x)), "srwm_backward_detached")
    return grad_x, gWy


class SrwmLayer(torch.autograd.Function):
    """Autograd boundary of :func:`srwm_layer`."""

    @staticmethod
    def forward(ctx, x, W_y, W_q, W_k, w_b, s_y, s_q, s_k, s_b, done, input_softmax, detach_state):
        base = (W_y, W_q, W_k, w_b)
        shift = None if s_y is None else (s_y, s_q, s_k, s_b)
        if done is not None and not detach_state:
            raise ValueError("done (in-kernel state reset) needs detach_state=True: the reverse-time "
                             "backward cannot cross a reset")
        need = any(ctx.needs_input_grad[:9])
        ctx.set_materialize_grads(False)     # unused outputs arrive as None, not as zero tensors
        out, shift_out, saved = srwm_layer_forward(x, base, shift, done, input_softmax, save=need)
        ctx.cfg = (input_softmax, detach_state, shift is not None, done is not None)
        if need:
            if detach_state:
                _, k, beta, yd, _, _, _ = saved
                keep = [x, k, beta, yd, W_y]
                if shift is not None:
                    keep.append(s_y)
                if done is not None:
                    keep.append(done)
                ctx.save_for_backward(*keep)
            else:
                ctx.save_for_backward(x, *saved, *base, *shift_out)
        if detach_state:
            ctx.mark_non_differentiable(*shift_out)
        ctx.base_shapes = [b.shape for b in base]
        return (out, *shift_out)

    @staticmethod
    def backward(ctx, grad_out, g_sy, g_sq, g_sk, g_sb):
        input_softmax, detach_state, has_shift, has_done = ctx.cfg
        if detach_state:
            t = list(ctx.saved_tensors)
            x, k, beta, yd, W_y = t[:5]
            rest = t[5:]
            s_y = rest.pop(0) if has_shift else None
            done = rest.pop(0) if has_done else None
            if grad_out is None:
                grad_out = torch.zeros_like(x)
            gx, gWy = srwm_backward_detached(x, (None, k, beta, yd, None, None, None), grad_out, W_y, s_y, done,
                                             input_softmax)
            need = ctx.needs_input_grad
            gb = [None] * 4
            if need[1]:
                gb[0] = _reduce_to(gWy, ctx.base_shapes[0])
            for i in (1, 2, 3):     # the detached state passes no gradient to the other three
                if need[1 + i]:
                    gb[i] = torch.zeros(ctx.base_shapes[i], device=x.device, dtype=torch.float32)
            return (gx if need[0] else None, *gb, None, None, None, None, None, None, None)
        t = ctx.saved_tensors
        x, saved, base, shift_out = t[0], t[1:8], t[8:12], t[12:16]
        if grad_out is None:
            grad_out = torch.zeros_like(x)
        g_out_state = (g_sy, g_sq, g_sk, g_sb)
        res = srwm_layer_backward(x, saved, grad_out, base, shift_out, g_out_state, input_softmax)
        gx, gW = res[0], res[1:]
        need = ctx.needs_input_grad
        gb = [None] * 4
        for i in range(4):
            if need[1 + i]:
                gb[i] = _reduce_to(gW[i], ctx.base_shapes[i])
                if g_out_state[i] is not None:      # shift_out = W_L - base
                    gb[i] = gb[i] - _reduce_to(g_out_state[i].to(torch.float32).contiguous(), ctx.base_shapes[i])
        gs = [gW[i] if (has_shift and need[5 + i]) else None for i in range(4)]
        return (gx if need[0] else None, *gb, *gs, None, None, None)


def _reduce_to(g, shape):
    """Per-sample gradient [N,H,E,.] -> gradient of a slow weight of ``shape`` ([1,...]: batch sum)."""
    if shape[0] == g.shape[0] and shape[0] != 1:
        return g
    return reduce_batch(g).view(shape)


def srwm_layer(x, W_y, W_q, W_k, w_b, shift=None, done=None, input_softmax=True, detach_state=False):
    """See the module docstring.  Returns (out, (shift_W_y, shift_W_q, shift_W_k, shift_w_b))."""
    s = (None, None, None, None) if shift is None else tuple(shift)
    if not (torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (x, W_y, W_q, W_k, w_b, *s))):
        # nothing to differentiate (the actors' path): skip the autograd machinery altogether
        if done is not None and not detach_state:
            raise ValueError("done (in-kernel state reset) needs detach_state=True")
        out, shift_out, _ = srwm_layer_forward(x, (W_y, W_q, W_k, w_b), shift, done, input_softmax, save=False)
        return out, tuple(shift_out)
    res = SrwmLayer.apply(x, W_y, W_q, W_k, w_b, *s, done, bool(input_softmax), bool(detach_state))
    return res[0], tuple(res[1:])


# ---------------------------------------------------------------------------------------
# delta rule on the packed slow-net rows
# ---------------------------------------------------------------------------------------

def _packed_ok(t):
    return t.stride(3) == 1 or t.size(3) == 1


def delta_packed_forward(qkvb, W, norm_eps=0.0, zero_init=False, save=True):
    """qkvb [N,H,L,3E+1] view of the raw rows (any strides, contiguous rows); W [N,H,E,E] fp32
    in/out (not read with ``zero_init``).  Returns (out [N,H,L,E], saved or None)."""
    _require_cuda(qkvb, W)
    N, H, Ln, RS = qkvb.shape
    E = (RS - 1) // 3
    assert RS == 3 * E + 1 and W.shape == (N, H, E, E)
    dt = _io_dtype(qkvb)
    xs = qkvb.detach()
    if not _packed_ok(xs):
        xs = xs.contiguous()
    assert _state_ok(W), "the fast-weight state must be a dense fp32 tensor"
    dev = qkvb.device
    out = _like(xs, E)
    a = L.DeltaPackedFwdArgs()
    a.N, a.H, a.L, a.E = N, H, Ln, E
    a.io_dtype = dt
    a.flags = (0 if save else L.FLAG_NO_SAVE) | (L.FLAG_ZERO_INIT if zero_init else 0)
    a.variant = 0
    a.norm_eps = float(norm_eps)
    a.qkvb = _seq_desc(xs)
    a.W = _state_desc(W)
    a.out = _seq_desc(out)
    saved = None
    if save:
        v_old, v_ins = torch.empty((2, N, H, Ln, E), device=dev, dtype=torch.float32).unbind(0)
        saved = (v_old, v_ins)
        a.v_old, a.v_insert = _seq_desc(v_old), _seq_desc(v_ins)
    else:
        a.v_old = a.v_insert = _NULL_SEQ
    if Ln == 0 and zero_init:
        W.zero_()
    with torch.cuda.device(dev):
        L.check(L.load().srwm_b200_delta_packed_forward(C.byref(a), _stream(qkvb)), "delta_packed_forward")
    return out, saved


def delta_packed_backward(qkvb, saved, grad_out, W, norm_eps=0.0, want_grad_W0=False):
    """W holds W_L on entry and W_0 on return.  Returns (grad_qkvb laid out like qkvb, grad_W0 or None)."""
    _require_cuda(qkvb, grad_out, W)
    N, H, Ln, RS = qkvb.shape
    E = (RS - 1) // 3
    dt = _io_dtype(qkvb)
    v_old, v_ins = saved
    xs = qkvb.detach()
    if not _packed_ok(xs):
        xs = xs.contiguous()
    go = _seq(grad_out.detach().to(qkvb.dtype))
    dev = qkvb.device
    gx = torch.empty_like(xs)
    gW0 = torch.empty((N, H, E, E), device=dev, dtype=torch.float32) if want_grad_W0 else None
    a = L.DeltaPackedBwdArgs()
    a.N, a.H, a.L, a.E = N, H, Ln, E
    a.io_dtype = dt
    a.flags = 0
    a.variant = 0
    a.norm_eps = float(norm_eps)
    a.qkvb = _seq_desc(xs)
    a.v_old, a.v_insert = _seq_desc(v_old), _seq_desc(v_ins)
    a.grad_out = _seq_desc(go)
    a.W = _state_desc(W)
    a.grad_qkvb = _seq_desc(gx)
    a.grad_W0 = _state_desc(gW0) if want_grad_W0 else _NULL_STATE
    with torch.cuda.device(dev):
        L.check(L.load().srwm_b200_delta_packed_backward(C.byref(a), _stream(qkvb)), "delta_packed_backward")
    return gx, gW0


class DeltaLayer(torch.autograd.Function):
    """Autograd boundary of :func:`delta_layer` (no gradient for the state, as in
    ``DeltaFastWeight``, supervised_learning/fast_weight/__init__.py:96)."""

    @staticmethod
    def forward(ctx, qkvb, W, norm_eps, zero_init):
        need = ctx.needs_input_grad[0]
        out, saved = delta_packed_forward(qkvb, W, norm_eps, zero_init, save=need)
        ctx.norm_eps = norm_eps
        if need:
            ctx.save_for_backward(qkvb, *saved, W)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        qkvb, v_old, v_ins, W = ctx.saved_tensors
        gx, _ = delta_packed_backward(qkvb, (v_old, v_ins), grad_out, W, ctx.norm_eps)
        return gx, None, None, None


def delta_layer(qkvb, W, norm_eps=0.0, zero_init=False):
    """See the module docstring.  qkvb: [N,H,L,3E+1] view of the slow net's rows; W: [N,H,E,E]
    fp32 state, left holding the final fast weights (W_0 again after the backward)."""
    return DeltaLayer.apply(qkvb, W, float(norm_eps), bool(zero_init))
