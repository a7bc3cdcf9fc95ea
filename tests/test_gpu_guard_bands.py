"""Out-of-bounds and unwritten-output checks without a sanitizer.

Every tensor a kernel WRITES (outputs, saved activations, gradients, in/out state) is carved out
of a byte buffer filled with 0xFF, with 256 bytes of that fill kept on both sides.  0xFF bytes
read as NaN in fp32 and bf16, so after the call

* the guard bands must still be 0xFF everywhere (nothing was written outside the tensor), and
* no NaN may be left inside (every element was written),

and the results must equal, bit for bit, those of the ordinary call path on the same inputs.
Sequence lengths sit around the kernels' time-chunk length T (T-1, T, T+1, 2T+1) where the
staging and flushing code has its edge cases; views are dense and time-major strided
(``[L, N, H, E]`` memory order, as the layers pass them).  Calls go through the C ABI.
"""
import ctypes as C

import pytest
import torch

from conftest import delta_inputs, srwm_inputs

pytestmark = pytest.mark.gpu
GUARD = 256


def _dev():
    return torch.device("cuda", 0)


class Guarded:
    """Tensors carved out of 0xFF-filled buffers with guard bands."""

    def __init__(self):
        self.items = []

    def make(self, shape, dtype, time_major=False):
        d = _dev()
        es = torch.empty((), dtype=dtype).element_size()
        n = 1
        for s in shape:
            n *= s
        buf = torch.full((GUARD + n * es + GUARD,), 0xFF, dtype=torch.uint8, device=d)
        inner = buf[GUARD:GUARD + n * es].view(dtype)
        if time_major and len(shape) == 4:
            N, H, L, X = shape
            t = inner.view(L, N, H, X).permute(1, 2, 0, 3)
        else:
            t = inner.view(*shape)
        self.items.append((buf, n * es, t))
        return t

    def check(self):
        for buf, nb, t in self.items:
            assert bool((buf[:GUARD] == 0xFF).all()), "write below a tensor"
            assert bool((buf[GUARD + nb:] == 0xFF).all()), "write above a tensor"
            assert not bool(torch.isnan(t.float()).any()), "an output element was never written"


def _call_srwm(x, Ws, go, g, time_major):
    from srwm_b200 import _lib as L
    from srwm_b200.ops import _seq_desc, _state_desc, _stream
    N, H, Ln, E = x.shape
    dt = x.dtype
    f32 = torch.float32
    out = g.make((N, H, Ln, E), dt, time_major)
    saved = [g.make((N, H, Ln, E), f32) for _ in range(2)] + [g.make((N, H, Ln, 4), f32)] + \
            [g.make((N, H, Ln, E), f32) for _ in range(3)] + [g.make((N, H, Ln, 4), f32)]
    W = [g.make(w.shape, f32) for w in Ws]
    for a, b in zip(W, Ws):
        a.copy_(b)
    a = L.SrwmFwdArgs()
    a.N, a.H, a.L, a.E = N, H, Ln, E
    a.io_dtype = L.BF16 if dt == torch.bfloat16 else L.F32
    a.flags, a.variant = 0, 0
    a.x = _seq_desc(x)
    a.W_y, a.W_q, a.W_k, a.w_b = (_state_desc(t) for t in W)
    a.out = _seq_desc(out)
    a.q, a.k, a.beta, a.y_diff, a.q_diff, a.k_diff, a.beta_diff = (_seq_desc(t) for t in saved)
    L.check(L.load().srwm_b200_srwm_forward(C.byref(a), _stream(x)), "srwm_forward")
    gx = g.make((N, H, Ln, E), dt, time_major)
    gW = [g.make(w.shape, f32) for w in Ws]
    b = L.SrwmBwdArgs()
    b.N, b.H, b.L, b.E = N, H, Ln, E
    b.io_dtype, b.flags, b.variant = a.io_dtype, L.FLAG_RESTORE_STATE, 0
    b.x = _seq_desc(x)
    b.q, b.k, b.beta, b.y_diff, b.q_diff, b.k_diff, b.beta_diff = (_seq_desc(t) for t in saved)
    b.grad_out = _seq_desc(go)
    b.W_y, b.W_q, b.W_k, b.w_b = (_state_desc(t) for t in W)
    b.grad_x = _seq_desc(gx)
    b.grad_W_y, b.grad_W_q, b.grad_W_k, b.grad_w_b = (_state_desc(t) for t in gW)
    L.check(L.load().srwm_b200_srwm_backward(C.byref(b), _stream(x)), "srwm_backward")
    torch.cuda.synchronize()
    return out, saved, gx, gW, W


def _put(t, dt, time_major):
    d = _dev()
    if time_major:
        return t.permute(2, 0, 1, 3).contiguous().to(d, dt).permute(1, 2, 0, 3)
    return t.to(d, dt)


@pytest.mark.parametrize("time_major", [False, True])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E", [16, 32, 64])
@pytest.mark.parametrize("L", [15, 16, 17, 33])
def test_srwm_writes_exactly_its_outputs(E, L, dt, time_major):
    import srwm_b200 as sb
    N, H = 2, 3
    x, Ws, go = srwm_inputs(N, H, L, E, 31)
    xd, god = _put(x, dt, time_major), _put(go, dt, time_major)
    Wd = [w.to(_dev()) for w in Ws]
    g = Guarded()
    out, saved, gx, gW, W0 = _call_srwm(xd, Wd, god, g, time_major)
    g.check()
    # the ordinary path on the same inputs: identical bits
    W2 = [w.clone() for w in Wd]
    out2, saved2 = sb.srwm_forward(xd, *W2)
    grads2 = sb.srwm_backward(xd, saved2, god, *W2, restore_state=True)
    assert torch.equal(out, out2) and torch.equal(gx, grads2[0])
    for a, b in zip(saved, saved2):
        assert torch.equal(a, b)
    for a, b in zip(gW, grads2[1:]):
        assert torch.equal(a, b)
    for a, b in zip(W0, W2):
        assert torch.equal(a, b)


def _call_delta(Q, K, V, B, W0, go, g, time_major):
    from srwm_b200 import _lib as L
    from srwm_b200.ops import _seq_desc, _state_desc, _stream
    N, H, Ln, E = Q.shape
    dt = Q.dtype
    f32 = torch.float32
    out = g.make((N, H, Ln, E), dt, time_major)
    v_old, v_ins = g.make((N, H, Ln, E), f32), g.make((N, H, Ln, E), f32)
    W = g.make(W0.shape, f32)
    W.copy_(W0)
    a = L.DeltaFwdArgs()
    a.N, a.H, a.L, a.E, a.M = N, H, Ln, E, E
    a.io_dtype = L.BF16 if dt == torch.bfloat16 else L.F32
    a.flags, a.variant = 0, 0
    a.Q, a.K, a.V, a.beta = _seq_desc(Q), _seq_desc(K), _seq_desc(V), _seq_desc(B)
    a.W = _state_desc(W)
    a.out, a.v_old, a.v_insert = _seq_desc(out), _seq_desc(v_old), _seq_desc(v_ins)
    L.check(L.load().srwm_b200_delta_forward(C.byref(a), _stream(Q)), "delta_forward")
    gQ, gK, gV = (g.make((N, H, Ln, E), dt, time_major) for _ in range(3))
    gB = g.make((N, H, Ln, 1), dt)
    gW0 = g.make(W0.shape, f32)
    b = L.DeltaBwdArgs()
    b.N, b.H, b.L, b.E, b.M = N, H, Ln, E, E
    b.io_dtype, b.flags, b.variant = a.io_dtype, 0, 0
    b.Q, b.K, b.V, b.beta = a.Q, a.K, a.V, a.beta
    b.v_old, b.v_insert, b.grad_out = _seq_desc(v_old), _seq_desc(v_ins), _seq_desc(go)
    b.W = _state_desc(W)
    b.grad_Q, b.grad_K, b.grad_V, b.grad_beta = _seq_desc(gQ), _seq_desc(gK), _seq_desc(gV), _seq_desc(gB)
    b.grad_W0 = _state_desc(gW0)
    L.check(L.load().srwm_b200_delta_backward(C.byref(b), _stream(Q)), "delta_backward")
    torch.cuda.synchronize()
    return out, (v_old, v_ins), (gQ, gK, gV, gB, gW0), W


@pytest.mark.parametrize("time_major", [False, True])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E", [16, 32, 64])
@pytest.mark.parametrize("L", [7, 8, 9, 15, 16, 17, 33])
def test_delta_writes_exactly_its_outputs(E, L, dt, time_major):
    import srwm_b200 as sb
    N, H = 2, 3
    Q, K, V, B, W0, go = delta_inputs(N, H, L, E, 32, "rand")
    Qd, Kd, Vd, god = (_put(t, dt, time_major) for t in (Q, K, V, go))
    Bd = B.to(_dev(), dt)
    g = Guarded()
    out, saved, grads, W = _call_delta(Qd, Kd, Vd, Bd, W0.to(_dev()), god, g, time_major)
    g.check()
    W2 = W0.to(_dev()).clone()
    out2, saved2 = sb.delta_forward(Qd, Kd, Vd, Bd, W2)
    grads2 = sb.delta_backward(Qd, Kd, Vd, Bd, saved2, god, W2, want_grad_W0=True)
    assert torch.equal(out, out2)
    for a, b in zip(saved, saved2):
        assert torch.equal(a, b)
    for a, b in zip(grads, grads2):
        assert torch.equal(a, b)
    assert torch.equal(W, W2)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E", [16, 64])
@pytest.mark.parametrize("Ln", [7, 9, 17])
def test_packed_delta_rows_write_exactly_their_outputs(E, Ln, dt):
    """The layer-level delta call on the slow net's raw rows (3E+1 values: rows start at odd element
    offsets and are staged as the 16-byte blocks covering them).  The packed GRADIENT rows are
    written with element stores next to each other, so a stray element would land in a neighbouring
    row, not in a guard band: the row buffer is checked against the ordinary path bit for bit."""
    from srwm_b200 import _lib as L
    from srwm_b200 import layer_ops as lo
    from srwm_b200.ops import _seq_desc, _state_desc, _stream
    d = _dev()
    N, H = 2, 3
    RS = 3 * E + 1
    g0 = torch.Generator().manual_seed(33)
    raw = torch.randn(Ln, N, H * RS, generator=g0).to(d, dt)
    rows = raw.view(Ln, N, H, RS).permute(1, 2, 0, 3)
    go = torch.randn(N, H, Ln, E, generator=g0).to(d, dt)
    g = Guarded()
    out = g.make((N, H, Ln, E), dt, True)
    v_old, v_ins = g.make((N, H, Ln, E), torch.float32), g.make((N, H, Ln, E), torch.float32)
    W = g.make((N, H, E, E), torch.float32)
    a = L.DeltaPackedFwdArgs()
    a.N, a.H, a.L, a.E = N, H, Ln, E
    a.io_dtype = L.BF16 if dt == torch.bfloat16 else L.F32
    a.flags, a.variant, a.norm_eps = L.FLAG_ZERO_INIT, 0, 0.0
    a.qkvb, a.W = _seq_desc(rows), _state_desc(W)
    a.out, a.v_old, a.v_insert = _seq_desc(out), _seq_desc(v_old), _seq_desc(v_ins)
    L.check(L.load().srwm_b200_delta_packed_forward(C.byref(a), _stream(rows)), "packed forward")
    graw = g.make((Ln, N, H * RS), dt)
    grows = graw.view(Ln, N, H, RS).permute(1, 2, 0, 3)
    b = L.DeltaPackedBwdArgs()
    b.N, b.H, b.L, b.E = N, H, Ln, E
    b.io_dtype, b.flags, b.variant, b.norm_eps = a.io_dtype, 0, 0, 0.0
    b.qkvb, b.v_old, b.v_insert, b.grad_out = a.qkvb, a.v_old, a.v_insert, _seq_desc(go)
    b.W, b.grad_qkvb = _state_desc(W), _seq_desc(grows)
    b.grad_W0 = L.State(None, 0, 0)
    L.check(L.load().srwm_b200_delta_packed_backward(C.byref(b), _stream(rows)), "packed backward")
    torch.cuda.synchronize()
    g.check()
    W2 = torch.empty(N, H, E, E, device=d)
    out2, saved2 = lo.delta_packed_forward(rows, W2, 0.0, True)
    res2 = lo.delta_packed_backward(rows, saved2, go, W2, 0.0)
    assert torch.equal(out, out2) and torch.equal(v_old, saved2[0]) and torch.equal(v_ins, saved2[1])
    assert torch.equal(grows, res2[0])
    assert float(W.abs().max()) < 1e-5 and torch.equal(W, W2)
