"""GPU parity tests: the CUDA kernels, called through the C ABI, against the CPU oracle.

Tolerances (whole-tensor max error over max magnitude): forward <= 1e-4, gradients <= 1e-3
for fp32 activations.  With bf16 activations the outputs that are themselves rounded to
bf16 carry that rounding (<= 2^-8 relative); everything kept in fp32 (saved activations,
state, state gradients) is held to the fp32 bounds.
"""
import os

import pytest
import torch

import srwm_oracle as orc
from conftest import GOLDEN, delta_inputs, srwm_inputs

pytestmark = pytest.mark.gpu

FWD_TOL, GRAD_TOL = 1e-4, 1e-3
BF16_TOL = 8e-3


def _err(a, b, floor=1e-3):
    """Both views of the error, the larger one: whole-tensor max|err| / max|ref|, and the
    reference's element-wise relative error on every element above ``floor`` times the tensor's
    largest magnitude.  Gradients (1e-3): every element above a thousandth of the largest.
    Forward tensors (1e-4, ``_errf``): every element above a hundredth -- an fp32 dot product of
    64 terms carries about 5e-7 of the tensor's scale, which already is 1e-4 of an element a
    two-hundredth of that scale (the saved q.W - k.W differences are the tightest case)."""
    return max(orc.rel_max(a, b), orc.rel_elem(a, b, floor))


def _errf(a, b):
    return _err(a, b, 1e-2)


def _sb():
    import srwm_b200 as sb
    return sb


def _nvar(op, E):
    from srwm_b200 import _lib as L
    return L.load().srwm_b200_num_variants(op, E)


def _dev():
    return torch.device("cuda", 0)


# ---------------------------------------------------------------------------------------
# the reference's own self-test cases (golden fixtures)
# ---------------------------------------------------------------------------------------

def test_srwm_reference_main_case():
    sb = _sb()
    g = torch.load(os.path.join(GOLDEN, "srwm_main_3x5x11x8.pt"))
    d = _dev()
    x = g["x"].to(d).requires_grad_()
    Ws = [g[k].to(d).requires_grad_() for k in ("W_y", "W_q", "W_k", "w_b")]
    out = sb.self_ref_v0(x, *[w.clone() for w in Ws])
    out.sum().backward()                       # the reference's loss (__init__.py:380)
    # the reference's metric and threshold, row by row as it does (__init__.py:229-233,370)
    assert orc.max_relative_error(out.detach().cpu(), g["out"]) < 1e-3
    assert orc.max_relative_error(x.grad.cpu(), g["grad_x"]) < 1e-3
    for w, k in zip(Ws, ("grad_W_y", "grad_W_q", "grad_W_k", "grad_w_b")):
        assert orc.max_relative_error(w.grad.cpu(), g[k]) < 1e-3, k
        assert orc.rel_max(w.grad.cpu(), g[k]) < 1e-5, k


def test_delta_reference_main_case():
    sb = _sb()
    g = torch.load(os.path.join(GOLDEN, "delta_main_3x5x11x64.pt"))
    d = _dev()
    leaves = [g[k].to(d).requires_grad_() for k in ("Q", "K", "V", "beta")]
    W = torch.zeros(3, 5, 64, 64, device=d)
    out = sb.fast_weight_delta(*leaves, W)
    out.sum().backward()
    assert orc.max_relative_error(out.detach().cpu(), g["out"]) < 1e-3
    for t, k in zip(leaves, ("grad_Q", "grad_K", "grad_V", "grad_beta")):
        assert orc.max_relative_error(t.grad.cpu(), g[k]) < 1e-3, k
    assert float(W.abs().max()) < 1e-5         # backward restored W_0 = 0


# ---------------------------------------------------------------------------------------
# SRWM against the fp64 oracle
# ---------------------------------------------------------------------------------------

def _srwm_check(N, H, L, E, dtype=torch.float32, variant=(None, None), strided=False, state_grad=False,
                weight="normal", seed=11):
    sb = _sb()
    d = _dev()
    x, Ws, go = srwm_inputs(N, H, L, E, seed, weight)
    if dtype == torch.bfloat16:
        x, go = x.bfloat16().float(), go.bfloat16().float()
    gs = None
    if state_grad:
        g = torch.Generator().manual_seed(seed + 1)
        gs = [torch.randn(w.shape, generator=g) for w in Ws]
    f = orc.srwm_forward_explicit(x.double(), *[w.double() for w in Ws])
    r = orc.srwm_backward_explicit(x.double(), f["q"], f["k"], f["beta"], f["y_diff"], f["q_diff"], f["k_diff"],
                                   f["beta_diff"], go.double(), f["W_y"], f["W_q"], f["W_k"], f["w_b"],
                                   grad_state=[t.double() for t in gs] if gs else None)

    def put(t):
        if strided:   # memory order [L, N, H, E], as the layers pass it (layer.py:161-165)
            return t.permute(2, 0, 1, 3).contiguous().to(d, dtype).permute(1, 2, 0, 3)
        return t.to(d, dtype)

    xd, god = put(x), put(go)
    Wd = [w.to(d).clone() for w in Ws]
    out, saved = sb.srwm_forward(xd, *Wd, variant=variant[0])
    io_tol = BF16_TOL if dtype == torch.bfloat16 else FWD_TOL
    assert _errf(out.float().cpu(), f["out"]) < io_tol
    for t, k in zip(saved, ("q", "k", "beta", "y_diff", "q_diff", "k_diff", "beta_diff")):
        assert _errf(t.cpu(), f[k]) < FWD_TOL, k
    for t, k in zip(Wd, ("W_y", "W_q", "W_k", "w_b")):
        assert _errf(t.cpu(), f[k]) < FWD_TOL, "final " + k
    grads = sb.srwm_backward(xd, saved, god, *Wd, grad_state=[t.to(d) for t in gs] if gs else None,
                             restore_state=True, variant=variant[1])
    gx_tol = BF16_TOL if dtype == torch.bfloat16 else GRAD_TOL
    assert _err(grads[0].float().cpu(), r[0]) < gx_tol
    for t, o, k in zip(grads[1:], r[1:5], ("gW_y", "gW_q", "gW_k", "gw_b")):
        assert _err(t.cpu(), o) < GRAD_TOL, k
    for t, o in zip(Wd, Ws):                   # reversal rebuilt the initial state
        assert _errf(t.cpu(), o) < FWD_TOL
    if gs:                                     # incoming state gradients are not modified
        pass


@pytest.mark.parametrize("E", [8, 16, 32, 64])
@pytest.mark.parametrize("L", [1, 2, 15, 16, 17, 50])
def test_srwm_parity_lengths(E, L):
    _srwm_check(2, 3, L, E)


@pytest.mark.parametrize("E", [8, 16, 32, 64])
def test_srwm_parity_all_variants(E):
    for vf in range(_nvar(0, E)):
        _srwm_check(2, 2, 35, E, variant=(vf, 0))
    for vb in range(_nvar(1, E)):
        _srwm_check(2, 2, 35, E, variant=(0, vb))


@pytest.mark.parametrize("E", [16, 64])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_srwm_parity_strided_views(E, dtype):
    _srwm_check(3, 2, 40, E, dtype=dtype, strided=True)


@pytest.mark.parametrize("E", [8, 32, 64])
def test_srwm_parity_state_gradient(E):
    _srwm_check(2, 2, 21, E, state_grad=True)


def test_srwm_parity_uniform_weights_reference_style():
    _srwm_check(3, 5, 11, 8, weight="uniform")


def test_srwm_config1_full_size():
    # SRWM single layer, B=4 H=4 L=64 d=16, W0 ~ N(0, 1/16) per head repeated over the batch
    sb = _sb()
    d = _dev()
    g = torch.Generator().manual_seed(1001)
    x = torch.randn(4, 4, 64, 16, generator=g)
    slow = [torch.randn(1, 4, 16, 16, generator=g) * 0.25 for _ in range(3)] + [torch.randn(1, 4, 16, 4, generator=g) * 0.25]
    go = torch.randn(4, 4, 64, 16, generator=g)
    xr = x.double().requires_grad_()
    sr = [w.double().requires_grad_() for w in slow]
    ref, _ = orc.srwm_loop(xr, *[w.repeat(4, 1, 1, 1) for w in sr])
    (ref * go.double()).sum().backward()
    xd = x.to(d).requires_grad_()
    sd = [w.to(d).requires_grad_() for w in slow]
    out = sb.self_ref_v0(xd, *[w.repeat(4, 1, 1, 1) for w in sd])
    (out * go.to(d)).sum().backward()
    assert orc.rel_max(out.detach().cpu(), ref.detach()) < FWD_TOL
    assert orc.rel_max(xd.grad.cpu(), xr.grad) < GRAD_TOL
    for a, b in zip(sd, sr):
        assert orc.rel_max(a.grad.cpu(), b.grad) < GRAD_TOL


def test_srwm_config3_operator_size():
    # the operator call of the few-shot stack: B=128 H=16 L=128 d=32 (2048 sequences);
    # a random subset of sequences is checked against the oracle (sequences are independent)
    sb = _sb()
    d = _dev()
    N, H, L, E = 128, 16, 128, 32
    x, Ws, go = srwm_inputs(N, H, L, E, seed=1003)
    xd, god = x.to(d), go.to(d)
    Wd = [w.to(d).clone() for w in Ws]
    out, saved = sb.srwm_forward(xd, *Wd)
    grads = sb.srwm_backward(xd, saved, god, *Wd)
    idx = torch.tensor([0, 17, 63, 127])
    f = orc.srwm_forward_explicit(x[idx].double(), *[w[idx].double() for w in Ws])
    r = orc.srwm_backward_explicit(x[idx].double(), f["q"], f["k"], f["beta"], f["y_diff"], f["q_diff"], f["k_diff"],
                                   f["beta_diff"], go[idx].double(), f["W_y"], f["W_q"], f["W_k"], f["w_b"])
    assert orc.rel_max(out.cpu()[idx], f["out"]) < FWD_TOL
    assert orc.rel_max(grads[0].cpu()[idx], r[0]) < GRAD_TOL
    for t, o in zip(grads[1:], r[1:5]):
        assert orc.rel_max(t.cpu()[idx], o) < GRAD_TOL


def test_srwm_stateful_autograd_and_carried_state():
    # carried state: two segments through stateful_self_ref_v0 equal one long sequence,
    # gradients flow through the returned state (learner-style unroll with carried W)
    sb = _sb()
    d = _dev()
    N, H, L, E = 2, 2, 24, 32
    x, Ws, go = srwm_inputs(N, H, L, E, seed=21)
    xr = x.double().requires_grad_()
    Wr = [w.double().requires_grad_() for w in Ws]
    ref, _ = orc.srwm_loop(xr, *Wr)
    (ref * go.double()).sum().backward()
    xd = x.to(d).requires_grad_()
    Wd = [w.to(d).requires_grad_() for w in Ws]
    o1, *st = sb.stateful_self_ref_v0(xd[:, :, :10], *[w.clone() for w in Wd])
    # the carried state goes into the next call as fresh tensors, as the layers do
    # (`state + W.repeat(...)`, supervised_learning/layer.py:167-172): a later call must not
    # overwrite the storage an earlier call saved for its backward
    o2, *_ = sb.stateful_self_ref_v0(xd[:, :, 10:], *[s + 0.0 for s in st])
    out = torch.cat([o1, o2], dim=2)
    (out * go.to(d)).sum().backward()
    assert orc.rel_max(out.detach().cpu(), ref.detach()) < FWD_TOL
    assert orc.rel_max(xd.grad.cpu(), xr.grad) < GRAD_TOL
    for a, b in zip(Wd, Wr):
        assert orc.rel_max(a.grad.cpu(), b.grad) < GRAD_TOL


def test_srwm_inplace_final_state_and_no_grad_path():
    sb = _sb()
    d = _dev()
    x, Ws, _ = srwm_inputs(3, 2, 1, 32, seed=31)       # actor-style single step
    f = orc.srwm_forward_explicit(x.double(), *[w.double() for w in Ws])
    Wd = [w.to(d).clone() for w in Ws]
    with torch.no_grad():
        out = sb.self_ref_v0(x.to(d), *Wd)
    assert orc.rel_max(out.cpu(), f["out"]) < FWD_TOL
    for t, k in zip(Wd, ("W_y", "W_q", "W_k", "w_b")):
        assert orc.rel_max(t.cpu(), f[k]) < FWD_TOL
    # 100 consecutive single steps with the state carried equal one 100-step call
    x, Ws, _ = srwm_inputs(2, 2, 100, 32, seed=32)
    f = orc.srwm_forward_explicit(x.double(), *[w.double() for w in Ws])
    Wd = [w.to(d).clone() for w in Ws]
    xd = x.to(d)
    outs = []
    with torch.no_grad():
        for t in range(100):
            outs.append(sb.self_ref_v0(xd[:, :, t:t + 1], *Wd))
    assert orc.rel_max(torch.cat(outs, 2).cpu(), f["out"]) < FWD_TOL


def test_srwm_non_dense_state_is_copied_back():
    sb = _sb()
    d = _dev()
    x, Ws, _ = srwm_inputs(2, 2, 9, 16, seed=41)
    f = orc.srwm_forward_explicit(x.double(), *[w.double() for w in Ws])
    big = torch.zeros(2, 2, 16, 32, device=d)
    Wy_view = big[..., ::2]                              # inner stride 2: not dense
    Wy_view.copy_(Ws[0].to(d))
    rest = [w.to(d).clone() for w in Ws[1:]]
    out, _ = sb.srwm_forward(x.to(d), Wy_view, *rest, save=False)
    assert orc.rel_max(out.cpu(), f["out"]) < FWD_TOL
    assert orc.rel_max(Wy_view.cpu(), f["W_y"]) < FWD_TOL


def test_srwm_empty_and_determinism():
    sb = _sb()
    d = _dev()
    Ws = [torch.zeros(0, 2, 8, 8, device=d) for _ in range(3)] + [torch.zeros(0, 2, 8, 4, device=d)]
    out, saved = sb.srwm_forward(torch.zeros(0, 2, 5, 8, device=d), *Ws)
    assert out.shape == (0, 2, 5, 8)
    x, Ws, go = srwm_inputs(4, 4, 70, 64, seed=51)
    res = []
    for _ in range(2):
        Wd = [w.to(d).clone() for w in Ws]
        out, saved = sb.srwm_forward(x.to(d), *Wd)
        grads = sb.srwm_backward(x.to(d), saved, go.to(d), *Wd)
        res.append([out] + list(grads))
    for a, b in zip(*res):
        assert torch.equal(a, b)                        # bitwise run-to-run


def test_srwm_long_sequence_reversal_drift():
    # L = 2048 at d=64, bf16 activations: the reversal must land back on W_0 and the
    # gradients of a subset of sequences must match the oracle
    sb = _sb()
    d = _dev()
    N, H, L, E = 4, 2, 2048, 64
    x, Ws, go = srwm_inputs(N, H, L, E, seed=61)
    x, go = x.bfloat16(), go.bfloat16()
    Wd = [w.to(d).clone() for w in Ws]
    out, saved = sb.srwm_forward(x.to(d), *Wd)
    grads = sb.srwm_backward(x.to(d), saved, go.to(d), *Wd, restore_state=True)
    for t, o in zip(Wd, Ws):
        assert orc.rel_max(t.cpu(), o) < 1e-4
    idx = torch.tensor([1])
    f = orc.srwm_forward_explicit(x[idx].double(), *[w[idx].double() for w in Ws])
    r = orc.srwm_backward_explicit(x[idx].double(), f["q"], f["k"], f["beta"], f["y_diff"], f["q_diff"], f["k_diff"],
                                   f["beta_diff"], go[idx].double(), f["W_y"], f["W_q"], f["W_k"], f["w_b"])
    assert orc.rel_max(out.float().cpu()[idx], f["out"]) < BF16_TOL
    assert orc.rel_max(grads[0].float().cpu()[idx], r[0]) < BF16_TOL
    for t, o in zip(grads[1:], r[1:5]):
        assert orc.rel_max(t.cpu()[idx], o) < GRAD_TOL


# ---------------------------------------------------------------------------------------
# delta rule against the fp64 oracle
# ---------------------------------------------------------------------------------------

def _delta_check(N, H, L, E, dtype=torch.float32, variant=(None, None), strided=False, w0="rand", seed=12):
    sb = _sb()
    d = _dev()
    Q, K, V, B, W0, go = delta_inputs(N, H, L, E, seed, w0)
    if dtype == torch.bfloat16:
        Q, K, V, B, go = (t.bfloat16().float() for t in (Q, K, V, B, go))
    f = orc.delta_forward_explicit(Q.double(), K.double(), V.double(), B.double(), W0.double())
    r = orc.delta_backward_explicit(Q.double(), K.double(), V.double(), B.double(), f["v_old"], f["v_insert"],
                                    go.double(), f["W"])

    def put(t):
        if strided:
            return t.permute(2, 0, 1, 3).contiguous().to(d, dtype).permute(1, 2, 0, 3)
        return t.to(d, dtype)

    Qd, Kd, Vd, Bd, god = (put(t) for t in (Q, K, V, B, go))
    Wd = W0.to(d).clone()
    out, saved = sb.delta_forward(Qd, Kd, Vd, Bd, Wd, variant=variant[0])
    io_tol = BF16_TOL if dtype == torch.bfloat16 else FWD_TOL
    assert _errf(out.float().cpu(), f["out"]) < io_tol
    assert _errf(saved[0].cpu(), f["v_old"]) < FWD_TOL
    assert _errf(saved[1].cpu(), f["v_insert"]) < FWD_TOL
    assert _errf(Wd.cpu(), f["W"]) < FWD_TOL
    gQ, gK, gV, gB, gW0 = sb.delta_backward(Qd, Kd, Vd, Bd, saved, god, Wd, want_grad_W0=True, variant=variant[1])
    g_tol = BF16_TOL if dtype == torch.bfloat16 else GRAD_TOL
    for t, o, k in zip((gQ, gK, gV, gB), r[:4], "QKVb"):
        assert _err(t.float().cpu(), o) < g_tol, k
    assert _err(gW0.cpu(), r[5]) < GRAD_TOL
    assert float((Wd.cpu().double() - W0.double()).abs().max()) < 1e-5


@pytest.mark.parametrize("E", [8, 16, 32, 64])
@pytest.mark.parametrize("L", [1, 7, 8, 9, 16, 17, 45])
def test_delta_parity_lengths(E, L):
    _delta_check(2, 3, L, E)


@pytest.mark.parametrize("E", [32, 64])
def test_delta_parity_all_variants(E):
    for vf in range(_nvar(2, E)):
        _delta_check(2, 2, 35, E, variant=(vf, 0))
    for vb in range(_nvar(3, E)):
        _delta_check(2, 2, 35, E, variant=(0, vb))


@pytest.mark.parametrize("E", [16, 64])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_delta_parity_strided_views(E, dtype):
    _delta_check(3, 2, 40, E, dtype=dtype, strided=True)


def test_delta_config2_full_size():
    # B=32 H=8 L=512 d=64, W0 = 0
    _delta_check(32, 8, 512, 64, w0="zero", seed=1002)


def test_delta_layer_style_views_misaligned_v():
    # q,k,v,beta split out of one [L,B,H,3d+1] projection as the layer does
    # (supervised_learning/layer.py:71-82): v rows start at odd float offsets, so the
    # host layer has to make it contiguous; results must not change
    sb = _sb()
    d = _dev()
    L_, B_, H_, E = 19, 2, 3, 16
    g = torch.Generator().manual_seed(71)
    qkvb = torch.randn(L_, B_, H_, 3 * E + 1, generator=g)
    hq, hk, hv, hb = torch.split(qkvb, (E, E, E, 1), -1)
    prep = lambda t: t.permute(1, 2, 0, 3)
    Q = torch.softmax(prep(hq), -1)
    K = torch.softmax(prep(hk), -1)
    V = prep(hv)
    Bt = torch.sigmoid(prep(hb))
    go = torch.randn(B_, H_, L_, E, generator=g)
    leaves_r = [t.double().detach().requires_grad_() for t in (Q, K, V, Bt)]
    ref, _ = orc.delta_loop(*leaves_r, torch.zeros(B_, H_, E, E, dtype=torch.float64))
    (ref * go.double()).sum().backward()
    qd = qkvb.to(d)
    hq, hk, hv, hb = torch.split(qd, (E, E, E, 1), -1)
    Vd = prep(hv).detach().requires_grad_()                # non-contiguous, misaligned rows
    Qd = torch.softmax(prep(hq), -1).detach().requires_grad_()
    Kd = torch.softmax(prep(hk), -1).detach().requires_grad_()
    Bd = torch.sigmoid(prep(hb)).detach().requires_grad_()
    W = torch.zeros(B_, H_, E, E, device=d)
    out = sb.fast_weight_delta(Qd, Kd, Vd, Bd, W)
    (out * go.to(d)).sum().backward()
    assert orc.rel_max(out.detach().cpu(), ref.detach()) < FWD_TOL
    for a, b in zip((Qd, Kd, Vd, Bd), leaves_r):
        assert orc.rel_max(a.grad.cpu(), b.grad) < GRAD_TOL


def test_delta_long_sequence_bf16():
    # L = 8192 at d=64 with bf16 activations: state after undoing 8192 updates returns to 0
    sb = _sb()
    d = _dev()
    N, H, L, E = 2, 2, 8192, 64
    Q, K, V, B, W0, go = delta_inputs(N, H, L, E, seed=81)
    Q, K, V, B, go = (t.bfloat16() for t in (Q, K, V, B, go))
    W = W0.to(d).clone()
    out, saved = sb.delta_forward(Q.to(d), K.to(d), V.to(d), B.to(d), W)
    f = orc.delta_forward_explicit(Q[:1].double(), K[:1].double(), V[:1].double(), B[:1].double(), W0[:1].double())
    assert orc.rel_max(out.float().cpu()[:1], f["out"]) < BF16_TOL
    assert orc.rel_max(W.cpu()[:1], f["W"]) < FWD_TOL
    grads = sb.delta_backward(Q.to(d), K.to(d), V.to(d), B.to(d), saved, go.to(d), W)
    r = orc.delta_backward_explicit(Q[:1].double(), K[:1].double(), V[:1].double(), B[:1].double(), f["v_old"],
                                    f["v_insert"], go[:1].double(), f["W"])
    for t, o in zip(grads[:4], r[:4]):
        assert orc.rel_max(t.float().cpu()[:1], o) < BF16_TOL
    assert float(W.abs().max()) < 1e-3 * float(f["W"].abs().max())


def test_delta_linearity_in_values():
    # with W0 = 0 the output is linear in v: out(a*v1 + v2) = a*out(v1) + out(v2)
    sb = _sb()
    d = _dev()
    Q, K, V1, B, W0, _ = delta_inputs(8, 8, 300, 64, seed=91)
    V2 = torch.randn(V1.shape, generator=torch.Generator().manual_seed(92))

    def run(V):
        W = W0.to(d).clone()
        out, _ = sb.delta_forward(Q.to(d), K.to(d), V.to(d), B.to(d), W, save=False)
        return out.double()

    lhs = run(2.5 * V1 + V2)
    rhs = 2.5 * run(V1) + run(V2)
    assert orc.rel_max(lhs, rhs) < FWD_TOL


def test_reduce_batch_matches_sum():
    sb = _sb()
    d = _dev()
    g = torch.randn(37, 4, 16, 52, device=d)
    got = sb.reduce_batch(g)
    assert orc.rel_max(got.cpu(), g.double().sum(0).cpu()) < 1e-5
    acc = torch.ones(4, 16, 52, device=d)
    sb.reduce_batch(g, acc, accumulate=True)
    assert orc.rel_max(acc.cpu(), (g.double().sum(0) + 1).cpu()) < 1e-5


def test_full_size_sweep_config_subset():
    # the scale-sweep SRWM shape (H=16, d=64, L=2048, bf16) at a reduced batch; two
    # sequences are checked against the oracle
    sb = _sb()
    d = _dev()
    N, H, L, E = 16, 16, 2048, 64
    g = torch.Generator(device=d).manual_seed(1005)
    x = torch.randn(N, H, L, E, device=d, generator=g).bfloat16()
    go = torch.randn(N, H, L, E, device=d, generator=g).bfloat16()
    std = E ** -0.5
    slow = [torch.randn(1, H, E, E, device=d, generator=g) * std for _ in range(3)]
    slow.append(torch.randn(1, H, E, 4, device=d, generator=g) * std)
    Wd = [w.repeat(N, 1, 1, 1) for w in slow]
    out, saved = sb.srwm_forward(x, *Wd)
    grads = sb.srwm_backward(x, saved, go, *Wd)
    for n, h in ((0, 0), (15, 9)):
        xs = x[n:n + 1, h:h + 1].cpu().double()
        gos = go[n:n + 1, h:h + 1].cpu().double()
        Ws = [w[:, h:h + 1].cpu().double() for w in slow]
        f = orc.srwm_forward_explicit(xs, *Ws)
        r = orc.srwm_backward_explicit(xs, f["q"], f["k"], f["beta"], f["y_diff"], f["q_diff"], f["k_diff"],
                                       f["beta_diff"], gos, f["W_y"], f["W_q"], f["W_k"], f["w_b"])
        assert orc.rel_max(out[n:n + 1, h:h + 1].float().cpu(), f["out"]) < BF16_TOL
        assert orc.rel_max(grads[0][n:n + 1, h:h + 1].float().cpu(), r[0]) < BF16_TOL
        for t, o in zip(grads[1:], r[1:5]):
            assert orc.rel_max(t[n:n + 1, h:h + 1].cpu(), o) < GRAD_TOL


def test_layer_style_call_needs_no_layout_copies():
    # x as the SRWM layer passes it (supervised_learning/layer.py:161-165): the output comes
    # back in the same memory order, so the layer's transpose+reshape is a view
    sb = _sb()
    d = _dev()
    L_, B_, H_, E = 23, 3, 4, 32
    g = torch.Generator().manual_seed(77)
    h = torch.randn(L_, B_, H_ * E, generator=g)
    slow = [torch.randn(1, H_, E, E, generator=g) * E ** -0.5 for _ in range(3)] + [torch.randn(1, H_, E, 4, generator=g) * E ** -0.5]
    hd = h.to(d).requires_grad_()
    x = hd.reshape(L_, B_, H_, E).permute(1, 2, 0, 3)
    sd = [w.to(d).requires_grad_() for w in slow]
    out = sb.self_ref_v0(x, *[w.repeat(B_, 1, 1, 1) for w in sd])
    assert out.stride() == x.stride()
    back = out.transpose(1, 2).reshape(B_, L_, H_ * E)
    assert back.data_ptr() == out.data_ptr()
    y = back.transpose(0, 1)
    go = torch.randn(L_, B_, H_ * E, generator=g)
    (y * go.to(d)).sum().backward()
    hr = h.double().requires_grad_()
    sr = [w.double().requires_grad_() for w in slow]
    ref, _ = orc.srwm_loop(hr.reshape(L_, B_, H_, E).permute(1, 2, 0, 3), *[w.repeat(B_, 1, 1, 1) for w in sr])
    yr = ref.transpose(1, 2).reshape(B_, L_, H_ * E).transpose(0, 1)
    (yr * go.double()).sum().backward()
    assert orc.rel_max(y.detach().cpu(), yr.detach()) < FWD_TOL
    assert orc.rel_max(hd.grad.cpu(), hr.grad) < GRAD_TOL
    for a, b in zip(sd, sr):
        assert orc.rel_max(a.grad.cpu(), b.grad) < GRAD_TOL


def test_concurrent_calls_from_two_threads_and_streams():
    # the RL code calls the operator from a learner and an inference thread at the same time
    # (polybeast_learner.py:363,399): calls must be re-entrant and honour torch's current stream
    import threading
    sb = _sb()
    d = _dev()
    cases = []
    for seed, (N, H, L, E) in enumerate([(3, 4, 60, 32), (2, 8, 45, 16)]):
        x, Ws, go = srwm_inputs(N, H, L, E, seed=200 + seed)
        f = orc.srwm_forward_explicit(x.double(), *[w.double() for w in Ws])
        r = orc.srwm_backward_explicit(x.double(), f["q"], f["k"], f["beta"], f["y_diff"], f["q_diff"], f["k_diff"],
                                       f["beta_diff"], go.double(), f["W_y"], f["W_q"], f["W_k"], f["w_b"])
        cases.append((x.to(d), [w.to(d) for w in Ws], go.to(d), f, r))
    errors = []

    def worker(i):
        try:
            x, Ws, go, f, r = cases[i]
            stream = torch.cuda.Stream(device=d)
            with torch.cuda.stream(stream):
                for _ in range(20):
                    Wd = [w.clone() for w in Ws]
                    out, saved = sb.srwm_forward(x, *Wd)
                    grads = sb.srwm_backward(x, saved, go, *Wd)
                stream.synchronize()
            assert orc.rel_max(out.cpu(), f["out"]) < FWD_TOL
            for t, o in zip(grads, r[:5]):
                assert orc.rel_max(t.cpu(), o) < GRAD_TOL
        except Exception as e:  # noqa: BLE001
            errors.append((i, repr(e)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors


@pytest.mark.parametrize("E", [8, 16, 32, 64])
@pytest.mark.parametrize("strided", [False, True])
def test_bf16_activations_every_head_size(E, strided):
    _srwm_check(2, 3, 29, E, dtype=torch.bfloat16, strided=strided, state_grad=True)
    _delta_check(2, 3, 29, E, dtype=torch.bfloat16, strided=strided)


# ---------------------------------------------------------------------------------------
# empty sequences: the backward of a call with L = 0 launches, stages nothing and returns
# dL/dW_0 = dL/dW_L with the state untouched
# ---------------------------------------------------------------------------------------

@pytest.mark.parametrize("E", [8, 16, 32, 64])
def test_backward_of_an_empty_sequence(E):
    sb = _sb()
    d = _dev()
    N, H = 2, 3
    g = torch.Generator().manual_seed(3)
    x = torch.empty(N, H, 0, E, device=d)
    Ws = [torch.randn(N, H, E, E, generator=g).to(d) for _ in range(3)] + [torch.randn(N, H, E, 4, generator=g).to(d)]
    keep = [w.clone() for w in Ws]
    out, saved = sb.srwm_forward(x, *Ws)
    assert out.shape == (N, H, 0, E)
    gs = [torch.randn(w.shape, generator=g).to(d) for w in Ws]
    for state_grad in (None, gs):
        grads = sb.srwm_backward(x, saved, torch.empty_like(x), *Ws, grad_state=state_grad, restore_state=True)
        assert grads[0].shape == (N, H, 0, E)
        for i in range(4):
            want = gs[i] if state_grad is not None else torch.zeros_like(gs[i])
            assert torch.equal(grads[1 + i], want)
            assert torch.equal(Ws[i], keep[i])
    Q = torch.empty(N, H, 0, E, device=d)
    B = torch.empty(N, H, 0, 1, device=d)
    W = torch.randn(N, H, E, E, generator=g).to(d)
    W_keep = W.clone()
    out, saved = sb.delta_forward(Q, Q, Q, B, W)
    gQ, gK, gV, gB, gW0 = sb.delta_backward(Q, Q, Q, B, saved, torch.empty_like(Q), W, want_grad_W0=True)
    assert gQ.shape == (N, H, 0, E) and torch.equal(W, W_keep)
    assert float(gW0.abs().max()) == 0.0
    torch.cuda.synchronize()
