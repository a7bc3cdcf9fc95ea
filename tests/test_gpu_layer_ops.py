"""GPU parity tests of the layer-level SRWM calls (input softmax, un-repeated slow weights with
the state carried as a shift, in-kernel episode resets, detached-state backward) against the
CPU oracle of the reference layers' code around the operator (oracle/srwm_layer_oracle.py).

Tolerances as for the plain operator: forward <= 1e-4, gradients <= 1e-3 (whole-tensor max
error over max magnitude, fp32 activations); bf16 activations carry their own rounding.
"""
import pytest
import torch

import srwm_layer_oracle as lorc
import srwm_oracle as orc

pytestmark = pytest.mark.gpu

FWD_TOL, GRAD_TOL = 1e-4, 1e-3
BF16_TOL = 8e-3


def _dev():
    return torch.device("cuda", 0)


def _layer_inputs(N, H, L, E, seed, with_shift=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, H, L, E, generator=g)
    std = E ** -0.5
    base = [torch.randn(1, H, E, E, generator=g) * std for _ in range(3)]
    base.append(torch.randn(1, H, E, 4, generator=g) * std)
    shift = None
    if with_shift:
        shift = [torch.randn(N, H, E, E, generator=g) * 0.1 * std for _ in range(3)]
        shift.append(torch.randn(N, H, E, 4, generator=g) * 0.1 * std)
    go = torch.randn(N, H, L, E, generator=g)
    gs = [torch.randn(N, H, E, E, generator=g) for _ in range(3)] + [torch.randn(N, H, E, 4, generator=g)]
    return x, base, shift, go, gs


def _leaf(ts, dtype=torch.float64, device="cpu"):
    return [t.to(device=device, dtype=dtype).requires_grad_() for t in ts]


@pytest.mark.parametrize("E", [8, 16, 32, 64])
@pytest.mark.parametrize("with_shift", [False, True])
@pytest.mark.parametrize("input_softmax", [False, True])
def test_layer_bptt_parity(E, with_shift, input_softmax):
    from srwm_b200.layer_ops import srwm_layer
    N, H, L = 3, 2, 21
    x, base, shift, go, gs = _layer_inputs(N, H, L, E, 100 + E, with_shift)
    # oracle (fp64, autograd); the loss also reads the returned shift so that gradient flows into it
    xo = x.double().requires_grad_()
    bo = _leaf(base)
    so = _leaf(shift) if with_shift else None
    out_o, sh_o = lorc.srwm_layer(xo, bo, so, input_softmax)
    loss = (out_o * go.double()).sum() + sum((s * g.double()).sum() for s, g in zip(sh_o, gs))
    loss.backward()
    # kernels
    d = _dev()
    xd = x.to(d).requires_grad_()
    bd = _leaf(base, torch.float32, d)
    sd = _leaf(shift, torch.float32, d) if with_shift else None
    out, sh = srwm_layer(xd, *bd, shift=sd, input_softmax=input_softmax)
    assert orc.rel_max(out.detach().cpu(), out_o.detach()) < FWD_TOL
    for a, b in zip(sh, sh_o):
        assert a.shape == b.shape
        # the shift is a difference of two states: hold it to the tolerance at the states' scale
        assert float((a.detach().cpu() - b.detach()).abs().max()) < FWD_TOL * E ** -0.5
    loss_d = (out * go.to(d)).sum() + sum((s * g.to(d)).sum() for s, g in zip(sh, gs))
    loss_d.backward()
    assert orc.rel_max(xd.grad.cpu(), xo.grad) < GRAD_TOL
    for a, b in zip(bd, bo):
        assert a.grad.shape == b.grad.shape
        assert orc.rel_max(a.grad.cpu(), b.grad) < GRAD_TOL
    if with_shift:
        for a, b in zip(sd, so):
            assert orc.rel_max(a.grad.cpu(), b.grad) < GRAD_TOL


@pytest.mark.parametrize("E", [8, 16, 32, 64])
@pytest.mark.parametrize("input_softmax", [False, True])
def test_layer_unroll_detached_with_resets(E, input_softmax):
    from srwm_b200.layer_ops import srwm_layer
    N, H, T = 4, 2, 37
    x, base, shift, go, _ = _layer_inputs(N, H, T, E, 200 + E, True)
    g = torch.Generator().manual_seed(7)
    done = torch.rand(N, T, generator=g) < 0.12
    done[0, 0] = True            # a reset before the very first step
    done[1] = False              # a sample without any reset
    done[2, T - 1] = True        # and one at the last step
    xo = x.double().requires_grad_()
    bo = _leaf(base)
    out_o, sh_o = lorc.srwm_unroll_detached(xo, bo, [s.double() for s in shift], done, input_softmax)
    (out_o * go.double()).sum().backward()

    d = _dev()
    xd = x.to(d).requires_grad_()
    bd = _leaf(base, torch.float32, d)
    sd = [s.to(d) for s in shift]
    # the learner's mask is [T, B]: hand it in as the transposed view
    done_tb = done.t().contiguous().to(d)
    out, sh = srwm_layer(xd, *bd, shift=sd, done=done_tb.t(), input_softmax=input_softmax, detach_state=True)
    assert orc.rel_max(out.detach().cpu(), out_o.detach()) < FWD_TOL
    for a, b in zip(sh, sh_o):
        assert not a.requires_grad
        assert float((a.cpu() - b).abs().max()) < FWD_TOL * E ** -0.5
    (out * go.to(d)).sum().backward()
    assert orc.rel_max(xd.grad.cpu(), xo.grad) < GRAD_TOL
    assert orc.rel_max(bd[0].grad.cpu(), bo[0].grad) < GRAD_TOL
    for a, b in zip(bd[1:], bo[1:]):   # the detached state passes nothing to W_q, W_k, w_b
        assert float(a.grad.abs().max()) == 0.0
        assert b.grad is None or float(b.grad.abs().max()) == 0.0


def test_layer_detached_equals_one_step_calls_of_the_plain_operator():
    """The fused unroll against T one-step calls of the drop-in operator, composed as the
    reference layer composes them (torchbeast/layer.py:378-421), all on the GPU."""
    import srwm_b200 as sb
    from srwm_b200.layer_ops import srwm_layer
    N, H, T, E = 5, 4, 12, 32
    x, base, shift, go, _ = _layer_inputs(N, H, T, E, 321, True)
    d = _dev()
    done = (torch.rand(N, T, generator=torch.Generator().manual_seed(3)) < 0.2).to(d)
    xd = x.to(d).requires_grad_()
    bd = _leaf(base, torch.float32, d)
    out, sh = srwm_layer(xd, *bd, shift=[s.to(d) for s in shift], done=done, detach_state=True)
    (out * go.to(d)).sum().backward()

    x2 = x.to(d).requires_grad_()
    b2 = _leaf(base, torch.float32, d)
    st = [s.to(d) for s in shift]
    outs = []
    for t in range(T):
        nd = (~done[:, t]).float().view(N, 1, 1, 1)
        st = [nd * s for s in st]
        W = [s + b.repeat(N, 1, 1, 1) for s, b in zip(st, b2)]
        o = sb.self_ref_v0(torch.softmax(x2[:, :, t:t + 1], -1), *W)
        st = [w.detach() - b.detach().repeat(N, 1, 1, 1) for w, b in zip(W, b2)]
        outs.append(o)
    out2 = torch.cat(outs, 2)
    (out2 * go.to(d)).sum().backward()
    assert orc.rel_max(out.detach(), out2.detach()) < FWD_TOL
    assert orc.rel_max(xd.grad, x2.grad) < GRAD_TOL
    assert orc.rel_max(bd[0].grad, b2[0].grad) < GRAD_TOL
    for a, b in zip(sh, st):
        assert float((a - b).abs().max()) < FWD_TOL * E ** -0.5


@pytest.mark.parametrize("E", [16, 64])
def test_layer_style_views_bf16(E):
    """[L, B, H*d] bf16 activations handed in as the permuted view the layers build; the output
    comes back in the same memory order, so the layers' reshape stays a view."""
    from srwm_b200.layer_ops import srwm_layer
    B, H, L = 4, 2, 33
    g = torch.Generator().manual_seed(5)
    h = torch.randn(L, B, H * E, generator=g).bfloat16()
    _, base, shift, _, _ = _layer_inputs(B, H, L, E, 55, True)
    go = torch.randn(L, B, H * E, generator=g).bfloat16()
    xo = h.double().view(L, B, H, E).permute(1, 2, 0, 3).requires_grad_()
    bo = _leaf(base)
    out_o, sh_o = lorc.srwm_layer(xo, bo, [s.double() for s in shift], True)
    (out_o * go.double().view(L, B, H, E).permute(1, 2, 0, 3)).sum().backward()

    d = _dev()
    hd = h.to(d).requires_grad_()
    bd = _leaf(base, torch.float32, d)
    x = hd.view(L, B, H, E).permute(1, 2, 0, 3)
    out, sh = srwm_layer(x, *bd, shift=[s.to(d) for s in shift])
    res = out.transpose(1, 2).reshape(B, L, H * E).transpose(0, 1)     # layer.py:184-186
    assert res.data_ptr() == out.data_ptr() and res.is_contiguous()
    assert orc.rel_max(out.detach().float().cpu(), out_o.detach()) < BF16_TOL
    (res * go.to(d)).sum().backward()
    assert orc.rel_max(hd.grad.float().cpu().view(L, B, H, E).permute(1, 2, 0, 3), xo.grad) < BF16_TOL
    for a, b in zip(bd, bo):
        assert orc.rel_max(a.grad.cpu(), b.grad) < GRAD_TOL
    for a, b in zip(sh, sh_o):
        assert float((a.detach().cpu() - b.detach()).abs().max()) < FWD_TOL * E ** -0.5


def test_layer_per_sample_base_and_plain_entry_flag():
    """Slow weights given per sample ([N,H,E,.]) get per-sample gradients; the input-softmax
    flag alone (no base) goes through the plain entry points."""
    from srwm_b200 import _lib as L
    from srwm_b200 import ops
    from srwm_b200.layer_ops import srwm_layer
    N, H, Ln, E = 2, 3, 19, 16
    x, base, _, go, _ = _layer_inputs(N, H, Ln, E, 77, False)
    base = [b.repeat(N, 1, 1, 1) + 0.01 * torch.randn(N, *b.shape[1:]) for b in base]
    xo = x.double().requires_grad_()
    bo = _leaf(base)
    out_o, WL = orc.srwm_loop(torch.softmax(xo, -1), *bo)
    (out_o * go.double()).sum().backward()
    d = _dev()
    xd = x.to(d).requires_grad_()
    bd = _leaf(base, torch.float32, d)
    out, sh = srwm_layer(xd, *bd)
    (out * go.to(d)).sum().backward()
    assert orc.rel_max(out.detach().cpu(), out_o.detach()) < FWD_TOL
    assert orc.rel_max(xd.grad.cpu(), xo.grad) < GRAD_TOL
    for a, b in zip(bd, bo):
        assert a.grad.shape == b.grad.shape and orc.rel_max(a.grad.cpu(), b.grad) < GRAD_TOL
    # plain entry point with the flag: state in, final state out, as the reference operator
    import ctypes as C
    Wd = [b.to(d).clone() for b in base]
    xs = x.to(d)
    outp = torch.empty_like(xs)
    a = L.SrwmFwdArgs()
    a.N, a.H, a.L, a.E = N, H, Ln, E
    a.io_dtype = L.F32
    a.flags = L.FLAG_NO_SAVE | L.FLAG_INPUT_SOFTMAX
    a.x, a.out = ops._seq_desc(xs), ops._seq_desc(outp)
    a.W_y, a.W_q, a.W_k, a.w_b = (ops._state_desc(t) for t in Wd)
    L.check(L.load().srwm_b200_srwm_forward(C.byref(a), ops._stream(xs)), "srwm_forward")
    assert orc.rel_max(outp.cpu(), out_o.detach()) < FWD_TOL
    for t, o in zip(Wd, WL):
        assert orc.rel_max(t.cpu(), o.detach()) < FWD_TOL


def test_layer_done_needs_detached_state():
    from srwm_b200.layer_ops import srwm_layer
    d = _dev()
    x, base, _, _, _ = _layer_inputs(2, 2, 5, 8, 1, False)
    with pytest.raises(ValueError):
        srwm_layer(x.to(d), *[b.to(d) for b in base], done=torch.zeros(2, 5, dtype=torch.bool, device=d))


# ---------------------------------------------------------------------------------------
# the two layers against the reference layers' composition around the drop-in operator
# ---------------------------------------------------------------------------------------

def _composed_layer(layer, h, state, get_state, stateful, always_softmax=False):
    """What the reference layers compute (supervised_learning/layer.py:156-209,
    reinforcement_learning/torchbeast/layer.py:378-421), written with torch ops around the
    drop-in operator."""
    import srwm_b200 as sb
    slen, bsz, _ = h.shape
    H, E = layer.num_head, layer.dim_head
    x = h.reshape(slen, bsz, H, E)
    if always_softmax or layer.use_input_softmax:
        x = torch.softmax(x, dim=-1)
    x = x.permute(1, 2, 0, 3)
    Ws = [w.repeat(bsz, 1, 1, 1) for w in (layer.W_y, layer.W_q, layer.W_k, layer.w_b)]
    if state is not None:
        Ws = [s + w for s, w in zip(state, Ws)]
    if stateful:
        out, *Ws = sb.stateful_self_ref_v0(x, *Ws)
    else:
        out = sb.self_ref_v0(x, *Ws)
    out = out.transpose(1, 2).reshape(bsz, slen, H * E).transpose(0, 1)
    out = layer.drop(layer.out_linear(out))
    res = (layer.layer_norm(h) if getattr(layer, "use_ln", False) else h) + out
    if get_state:
        new = tuple(w - b.repeat(bsz, 1, 1, 1) for w, b in zip(Ws, (layer.W_y, layer.W_q, layer.W_k, layer.w_b)))
        return res, new
    return res


@pytest.mark.parametrize("use_ln,use_softmax,stateful", [(True, False, False), (False, True, True), (True, True, True)])
def test_srwm_layer_module_matches_composition(use_ln, use_softmax, stateful):
    from srwm_b200.layers import SRWMlayer
    d = _dev()
    torch.manual_seed(0)
    H, E, D, L, B = 4, 16, 64, 24, 3
    layer = SRWMlayer(H, E, D, 0.0, use_ln=use_ln, use_input_softmax=use_softmax, stateful=stateful).to(d)
    h = torch.randn(L, B, D, device=d)
    tgt = torch.randn(L, B, D, device=d)
    gs = [torch.randn(B, H, E, E, device=d) for _ in range(3)] + [torch.randn(B, H, E, 4, device=d)]
    st0 = [0.05 * torch.randn_like(g) for g in gs]

    def run(fused):
        layer.zero_grad()
        hh = h.clone().requires_grad_()
        st = [s.clone().requires_grad_() for s in st0]
        if fused:
            out, new = layer(hh, state=st, get_state=True)
        else:
            out, new = _composed_layer(layer, hh, st, True, stateful)
        loss = (out * tgt).sum()
        if stateful:
            loss = loss + sum((n * g).sum() for n, g in zip(new, gs))
        loss.backward()
        grads = [p.grad.clone() for p in layer.parameters()]
        return out.detach(), [n.detach() for n in new], hh.grad, [s.grad for s in st], grads

    o1, n1, gh1, gst1, gp1 = run(True)
    o2, n2, gh2, gst2, gp2 = run(False)
    assert orc.rel_max(o1, o2) < FWD_TOL
    for a, b in zip(n1, n2):
        assert float((a - b).abs().max()) < FWD_TOL * E ** -0.5
    assert orc.rel_max(gh1, gh2) < GRAD_TOL
    for a, b in zip(gst1, gst2):
        assert orc.rel_max(a, b) < GRAD_TOL
    for a, b, (name, _) in zip(gp1, gp2, layer.named_parameters()):
        assert orc.rel_max(a, b) < GRAD_TOL, name


def test_sr_layer_unroll_matches_the_learner_loop():
    from srwm_b200.layers import SRlayer
    d = _dev()
    torch.manual_seed(1)
    H, E, D, T, B = 8, 32, 256, 20, 6
    layer = SRlayer(H, E, D, 0.0).to(d)
    h = torch.randn(T, B, D, device=d)
    tgt = torch.randn(T, B, D, device=d)
    done = torch.rand(T, B, device=d) < 0.15
    st0 = [0.05 * torch.randn(B, H, E, E, device=d) for _ in range(3)] + [0.05 * torch.randn(B, H, E, 4, device=d)]

    layer.zero_grad()
    h1 = h.clone().requires_grad_()
    out1, s1 = layer.unroll(h1, done, [s.clone() for s in st0])
    (out1 * tgt).sum().backward()
    g1 = {n: p.grad.clone() for n, p in layer.named_parameters() if p.grad is not None}

    # reinforcement_learning/torchbeast_procgen/model.py:1180-1197 around the layer's own forward
    layer.zero_grad()
    h2 = h.clone().requires_grad_()
    st = [s.clone() for s in st0]
    outs = []
    for t in range(T):
        nd = (~done[t]).float().view(B, 1, 1, 1)
        st = [nd * s for s in st]
        o, st = _composed_layer(layer, h2[t:t + 1], st, True, False, always_softmax=True)
        st = [s.detach() for s in st]
        outs.append(o)
    out2 = torch.cat(outs, 0)
    (out2 * tgt).sum().backward()
    assert orc.rel_max(out1.detach(), out2.detach()) < FWD_TOL
    assert orc.rel_max(h1.grad, h2.grad) < GRAD_TOL
    for a, b in zip(s1, st):
        assert float((a - b).abs().max()) < FWD_TOL * E ** -0.5
    for n, p in layer.named_parameters():
        if n in ("W_q", "W_k", "w_b"):
            assert float(g1[n].abs().max()) == 0.0 and float(p.grad.abs().max()) < 1e-6
        elif p.grad is not None:
            assert orc.rel_max(g1[n], p.grad) < GRAD_TOL, n


# ---------------------------------------------------------------------------------------
# delta rule on the packed slow-net rows
# ---------------------------------------------------------------------------------------

@pytest.mark.parametrize("E", [8, 16, 32, 64])
@pytest.mark.parametrize("eps,zero_init", [(0.0, True), (1e-5, False)])
def test_delta_packed_layer_parity(E, eps, zero_init):
    from srwm_b200.layer_ops import delta_layer
    L, B, H = 29, 3, 2
    RS = 3 * E + 1
    g = torch.Generator().manual_seed(300 + E)
    raw = torch.randn(L, B, H * RS, generator=g)
    go = torch.randn(B, H, L, E, generator=g)
    W0 = torch.zeros(B, H, E, E) if zero_init else 0.1 * torch.randn(B, H, E, E, generator=g)
    ro = raw.double().requires_grad_()
    out_o, WL = lorc.delta_layer(ro.view(L, B, H, RS).permute(1, 2, 0, 3), W0.double(), eps)
    (out_o * go.double()).sum().backward()

    d = _dev()
    rd = raw.to(d).requires_grad_()
    W = torch.full((B, H, E, E), float("nan"), device=d) if zero_init else W0.to(d).clone()
    out = delta_layer(rd.view(L, B, H, RS).permute(1, 2, 0, 3), W, norm_eps=eps, zero_init=zero_init)
    res = out.transpose(1, 2).reshape(B, L, H * E).transpose(0, 1)       # layer.py:98-100 stays a view
    assert res.data_ptr() == out.data_ptr() and res.is_contiguous()
    assert orc.rel_max(out.detach().cpu(), out_o.detach()) < FWD_TOL
    assert orc.rel_max(W.cpu(), WL.detach()) < FWD_TOL                    # final fast weights left in W
    (out * go.to(d)).sum().backward()
    assert rd.grad.shape == raw.shape and rd.grad.is_contiguous()
    gk, go_ = rd.grad.cpu().view(L, B, H, RS), ro.grad.view(L, B, H, RS)
    for name, sl in (("q", slice(0, E)), ("k", slice(E, 2 * E)), ("v", slice(2 * E, 3 * E)), ("b", slice(3 * E, RS))):
        assert orc.rel_max(gk[..., sl], go_[..., sl]) < GRAD_TOL, name
    assert float((W.cpu() - W0).abs().max()) < 1e-5                       # the backward put W_0 back


@pytest.mark.parametrize("E", [16, 64])
def test_delta_packed_layer_bf16_rows_at_odd_offsets(E):
    """bf16 rows of 3E+1 values start at 2-byte offsets: staged as covering 16-byte blocks."""
    from srwm_b200.layer_ops import delta_layer
    L, B, H = 21, 2, 3
    RS = 3 * E + 1
    g = torch.Generator().manual_seed(400 + E)
    raw = torch.randn(L, B, H * RS, generator=g).bfloat16()
    go = torch.randn(B, H, L, E, generator=g).bfloat16()
    ro = raw.double().requires_grad_()
    out_o, _ = lorc.delta_layer(ro.view(L, B, H, RS).permute(1, 2, 0, 3), torch.zeros(B, H, E, E).double(), 1e-5)
    (out_o * go.double()).sum().backward()
    d = _dev()
    rd = raw.to(d).requires_grad_()
    W = torch.empty(B, H, E, E, device=d)
    out = delta_layer(rd.view(L, B, H, RS).permute(1, 2, 0, 3), W, norm_eps=1e-5, zero_init=True)
    assert out.dtype == torch.bfloat16
    assert orc.rel_max(out.detach().float().cpu(), out_o.detach()) < BF16_TOL
    (out * go.to(d)).sum().backward()
    assert orc.rel_max(rd.grad.float().cpu(), ro.grad) < BF16_TOL


def test_delta_packed_equals_the_layer_composition_on_gpu():
    """Against the layers' own sequence of torch ops around the drop-in operator
    (supervised_learning/layer.py:66-100), both on the GPU."""
    import srwm_b200 as sb
    from srwm_b200.layer_ops import delta_layer
    L, B, H, E = 40, 4, 4, 32
    RS = 3 * E + 1
    d = _dev()
    g = torch.Generator().manual_seed(9)
    raw = torch.randn(L, B, H * RS, generator=g).to(d)
    go = torch.randn(L, B, H * E, generator=g).to(d)
    r1 = raw.clone().requires_grad_()
    W1 = torch.empty(B, H, E, E, device=d)
    o1 = delta_layer(r1.view(L, B, H, RS).permute(1, 2, 0, 3), W1, zero_init=True)
    o1 = o1.transpose(1, 2).reshape(B, L, H * E).transpose(0, 1)
    (o1 * go).sum().backward()
    r2 = raw.clone().requires_grad_()
    q, k, v, b = torch.split(r2.view(L, B, H, RS), (E, E, E, 1), -1)
    b = torch.sigmoid(b)
    q, k, v, b = (t.permute(1, 2, 0, 3) for t in (q, k, v, b))
    q = torch.nn.functional.elu(q, 1.0, False) + 1.0
    k = torch.nn.functional.elu(k, 1.0, False) + 1.0
    q, k = q / q.sum(-1, keepdim=True), k / k.sum(-1, keepdim=True)
    W2 = torch.zeros(B, H, E, E, device=d)
    o2 = sb.fast_weight_delta(q, k, v, b, W2)
    o2 = o2.transpose(1, 2).reshape(B, L, H * E).transpose(0, 1)
    (o2 * go).sum().backward()
    assert orc.rel_max(o1.detach(), o2.detach()) < FWD_TOL
    assert orc.rel_max(r1.grad, r2.grad) < GRAD_TOL


def test_fast_ff_layer_modules_match_composition():
    import srwm_b200 as sb
    from srwm_b200.layers import FastFFlayer, FastFFlayerRL
    d = _dev()
    torch.manual_seed(2)
    H, E, D, L, B = 4, 16, 64, 19, 3
    F_ = torch.nn.functional
    for cls, eps in ((FastFFlayer, 0.0), (FastFFlayerRL, 1e-5)):
        layer = cls(H, E, D, 0.0).to(d)
        x = torch.randn(L, B, D, device=d)
        tgt = torch.randn(L, B, D, device=d)
        st0 = 0.1 * torch.randn(B, H, E, E, device=d)

        layer.zero_grad()
        x1 = x.clone().requires_grad_()
        if cls is FastFFlayer:
            o1, s1 = layer(x1), None
        else:
            o1, s1 = layer(x1, st0.clone())
        (o1 * tgt).sum().backward()
        g1 = [p.grad.clone() for p in layer.parameters()]

        layer.zero_grad()
        x2 = x.clone().requires_grad_()
        qkvb = layer.slow_net(layer.layer_norm(x2)).view(L, B, H, 3 * E + 1)
        q, k, v, b = torch.split(qkvb, (E, E, E, 1), -1)
        b = torch.sigmoid(b)
        q, k, v, b = (t.permute(1, 2, 0, 3) for t in (q, k, v, b))
        q, k = F_.elu(q, 1.0, False) + 1.0, F_.elu(k, 1.0, False) + 1.0
        q, k = q / (q.sum(-1, keepdim=True) + eps), k / (k.sum(-1, keepdim=True) + eps)
        W = torch.zeros(B, H, E, E, device=d) if cls is FastFFlayer else st0.clone()
        o2 = sb.fast_weight_delta(q, k, v, b, W)
        s2 = W.clone()
        o2 = x2 + layer.out_linear(o2.transpose(1, 2).reshape(B, L, H * E).transpose(0, 1))
        (o2 * tgt).sum().backward()
        assert orc.rel_max(o1.detach(), o2.detach()) < FWD_TOL
        assert orc.rel_max(x1.grad, x2.grad) < GRAD_TOL
        for a, p_ in zip(g1, layer.parameters()):
            assert orc.rel_max(a, p_.grad) < GRAD_TOL
        if s1 is not None:
            assert orc.rel_max(s1, s2) < FWD_TOL


def test_graphed_actor_step_matches_eager():
    """The CUDA-graph replay of an actor step (two SRlayer + feed-forward blocks, state updated in
    place) against the same stack called eagerly, over several steps with a reset in between."""
    import torch.nn as nn
    from srwm_b200.graphs import GraphedSRStep
    from srwm_b200.layers import SRlayer
    d = _dev()
    torch.manual_seed(4)
    H, E, D, B = 8, 32, 256, 12
    layers = [(SRlayer(H, E, D, 0.0).to(d), nn.Sequential(nn.LayerNorm(D), nn.Linear(D, D)).to(d)) for _ in range(2)]
    pre = nn.Linear(D + 1, D).to(d)
    st0 = [[0.05 * torch.randn(B, H, E, E, device=d) for _ in range(3)] + [0.05 * torch.randn(B, H, E, 4, device=d)]
           for _ in range(2)]
    xs = [torch.randn(1, B, D + 1, device=d) for _ in range(6)]
    step = GraphedSRStep(layers, st0, xs[0], pre=pre)
    st = [[t.clone() for t in s] for s in st0]
    mask = torch.zeros(B, dtype=torch.bool, device=d)
    mask[::3] = True
    with torch.no_grad():
        for i, x in enumerate(xs):
            if i == 3:                      # episode ends for a third of the samples
                step.reset(mask)
                st = [[t * (~mask).float().view(B, 1, 1, 1) for t in s] for s in st]
            got = step(x).clone()
            h = pre(x)
            for li, (sr, ff) in enumerate(layers):
                h, new = sr(h, st[li])
                st[li] = list(new)
                h = ff(h)
            assert orc.rel_max(got, h) < FWD_TOL, i
    for a, b in zip(step.state, st):
        for u, v in zip(a, b):
            assert float((u - v).abs().max()) < FWD_TOL * E ** -0.5


def test_layer_unroll_detached_bf16():
    from srwm_b200.layer_ops import srwm_layer
    N, H, T, E = 3, 2, 40, 64
    x, base, shift, go, _ = _layer_inputs(N, H, T, E, 777, True)
    x, go = x.bfloat16(), go.bfloat16()
    done = torch.rand(N, T, generator=torch.Generator().manual_seed(8)) < 0.1
    xo = x.double().requires_grad_()
    bo = _leaf(base)
    out_o, sh_o = lorc.srwm_unroll_detached(xo, bo, [s.double() for s in shift], done, True)
    (out_o * go.double()).sum().backward()
    d = _dev()
    xd = x.to(d).requires_grad_()
    bd = _leaf(base, torch.float32, d)
    out, sh = srwm_layer(xd, *bd, shift=[s.to(d) for s in shift], done=done.to(d), detach_state=True)
    (out * go.to(d)).sum().backward()
    assert orc.rel_max(out.detach().float().cpu(), out_o.detach()) < BF16_TOL
    assert orc.rel_max(xd.grad.float().cpu(), xo.grad) < BF16_TOL
    assert orc.rel_max(bd[0].grad.cpu(), bo[0].grad) < GRAD_TOL
    for a, b in zip(sh, sh_o):
        assert float((a.cpu() - b).abs().max()) < FWD_TOL * E ** -0.5


@pytest.mark.parametrize("dtype,lead", [(torch.float32, 1), (torch.float32, 3), (torch.bfloat16, 5), (torch.bfloat16, 7)])
def test_delta_packed_rows_at_every_misalignment(dtype, lead):
    """The packed rows may start anywhere on the element grid: shift the whole tensor by a few
    elements inside its allocation so that every (address mod 16) case of the block staging occurs."""
    from srwm_b200.layer_ops import delta_layer
    L, B, H, E = 18, 2, 3, 16
    RS = 3 * E + 1
    g = torch.Generator().manual_seed(500 + lead)
    raw = torch.randn(L, B, H * RS, generator=g).to(dtype)
    go = torch.randn(B, H, L, E, generator=g).to(dtype)
    ro = raw.double().requires_grad_()
    out_o, _ = lorc.delta_layer(ro.view(L, B, H, RS).permute(1, 2, 0, 3), torch.zeros(B, H, E, E).double(), 0.0)
    (out_o * go.double()).sum().backward()
    d = _dev()
    buf = torch.zeros(raw.numel() + 16, dtype=dtype, device=d)
    rd = buf[lead:lead + raw.numel()].view(L, B, H * RS)
    rd.copy_(raw)
    rd.requires_grad_()
    W = torch.empty(B, H, E, E, device=d)
    out = delta_layer(rd.view(L, B, H, RS).permute(1, 2, 0, 3), W, zero_init=True)
    (out * go.to(d)).sum().backward()
    tol_f, tol_g = (FWD_TOL, GRAD_TOL) if dtype == torch.float32 else (BF16_TOL, BF16_TOL)
    assert orc.rel_max(out.detach().float().cpu(), out_o.detach()) < tol_f
    assert orc.rel_max(rd.grad.float().cpu(), ro.grad) < tol_g


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_delta_packed_layer_large_grid_column_kernel(dtype):
    """With enough sequences to fill the GPU the packed d=64 forward runs in the column layout
    (one warp per sequence); same checks as for the small cases."""
    from srwm_b200.layer_ops import delta_layer
    L, B, H, E = 19, 40, 16, 64      # 640 sequences
    RS = 3 * E + 1
    g = torch.Generator().manual_seed(91)
    raw = torch.randn(L, B, H * RS, generator=g).to(dtype)
    go = torch.randn(B, H, L, E, generator=g).to(dtype)
    ro = raw.double().requires_grad_()
    out_o, WL = lorc.delta_layer(ro.view(L, B, H, RS).permute(1, 2, 0, 3), torch.zeros(B, H, E, E).double(), 1e-5)
    (out_o * go.double()).sum().backward()
    d = _dev()
    rd = raw.to(d).requires_grad_()
    W = torch.full((B, H, E, E), float("nan"), device=d)
    out = delta_layer(rd.view(L, B, H, RS).permute(1, 2, 0, 3), W, norm_eps=1e-5, zero_init=True)
    tol_f, tol_g = (FWD_TOL, GRAD_TOL) if dtype == torch.float32 else (BF16_TOL, BF16_TOL)
    assert orc.rel_max(out.detach().float().cpu(), out_o.detach()) < tol_f
    assert orc.rel_max(W.cpu(), WL.detach()) < FWD_TOL
    (out * go.to(d)).sum().backward()
    assert orc.rel_max(rd.grad.float().cpu(), ro.grad) < tol_g


def test_layer_call_at_scale_matches_plain_operator_composition():
    """Several waves of sequences, many chunks, bf16: the fused layer call against torch softmax +
    repeat + the plain operator (two different kernel instantiations of this library)."""
    import srwm_b200 as sb
    from srwm_b200.layer_ops import srwm_layer
    d = _dev()
    N, H, L, E = 80, 16, 300, 64
    g = torch.Generator(device=d).manual_seed(17)
    x = torch.randn(N, H, L, E, device=d, generator=g).bfloat16()
    go = torch.randn(N, H, L, E, device=d, generator=g).bfloat16()
    std = E ** -0.5
    base = [torch.randn(1, H, E, E, device=d, generator=g) * std for _ in range(3)]
    base.append(torch.randn(1, H, E, 4, device=d, generator=g) * std)
    shift = [0.05 * std * torch.randn(N, H, E, w.shape[-1], device=d, generator=g) for w in base]
    x1 = x.clone().requires_grad_()
    b1 = [b.clone().requires_grad_() for b in base]
    out1, sh1 = srwm_layer(x1, *b1, shift=shift)
    (out1.float() * go.float()).sum().backward()
    x2 = x.clone().float().requires_grad_()
    b2 = [b.clone().requires_grad_() for b in base]
    W = [s + b.repeat(N, 1, 1, 1) for s, b in zip(shift, b2)]
    out2 = sb.self_ref_v0(torch.softmax(x2, -1), *W)      # fp32 activations: the tighter of the two
    (out2 * go.float()).sum().backward()
    assert orc.rel_max(out1.detach().float(), out2.detach()) < BF16_TOL
    assert orc.rel_max(x1.grad.float(), x2.grad) < BF16_TOL
    for a, b in zip(b1, b2):
        assert orc.rel_max(a.grad, b.grad) < 2e-2      # bf16 activations feed a sum over 80 x 300 steps
    for a, w, b in zip(sh1, W, b2):
        assert float((a.detach() - (w.detach() - b.detach())).abs().max()) < 5e-3 * std


# ---------------------------------------------------------------------------------------
# batch reduction fused into the backward (srwm_b200_srwm_layer_backward_reduced)
# ---------------------------------------------------------------------------------------

@pytest.mark.parametrize("E", [16, 32, 64])
@pytest.mark.parametrize("N", [1, 5, 64, 65, 130])
def test_fused_batch_reduction_matches_the_separate_one(E, N):
    """The slow-weight gradients formed inside the backward kernel (last CTA of a group of samples
    adds the group, last group of a head adds the groups) against the batch sum of the per-sample
    gradients in float64; per-sample outputs unchanged; two calls in a row (the counters return to
    zero), accumulation, and bitwise repeatability."""
    from srwm_b200 import layer_ops as lo
    d = torch.device("cuda", 0)
    H, L_ = 3, 20
    g = torch.Generator().manual_seed(100 + N + E)
    x = torch.randn(N, H, L_, E, generator=g).to(d)
    go = torch.randn(N, H, L_, E, generator=g).to(d)
    std = E ** -0.5
    base = [(torch.randn(1, H, E, w, generator=g) * std).to(d) for w in (E, E, E, 4)]
    out, shift_out, saved = lo.srwm_layer_forward(x, base, None, None, True)
    plain = lo.srwm_layer_backward(x, saved, go, base, shift_out, None, True)
    want = [t.double().sum(0, keepdim=True) for t in plain[1:]]
    dst = [torch.full((1, H, E, w), float("nan"), device=d) for w in (E, E, E, 4)]
    res = lo.srwm_layer_backward(x, saved, go, base, shift_out, None, True, reduce_into=dst)
    for a, b in zip(res, plain):
        assert torch.equal(a, b)                       # grad_x and the per-sample gradients: same bits
    for a, b in zip(dst, want):
        assert orc.rel_max(a.cpu(), b.cpu()) < 1e-5
    first = [t.clone() for t in dst]
    lo.srwm_layer_backward(x, saved, go, base, shift_out, None, True, reduce_into=dst)
    for a, b in zip(dst, first):
        assert torch.equal(a, b)                       # second call: same bits (fixed summation order)
    lo.srwm_layer_backward(x, saved, go, base, shift_out, None, True, reduce_into=dst, accumulate=True)
    for a, b in zip(dst, want):
        assert orc.rel_max(a.cpu(), 2 * b.cpu()) < 1e-5
    torch.cuda.synchronize()


def test_fused_batch_reduction_rejects_bad_scratch():
    import ctypes as C
    from srwm_b200 import _lib as L
    lib = L.load()
    assert lib.srwm_b200_srwm_reduce_scratch_bytes(130, 3, 64) > lib.srwm_b200_srwm_reduce_scratch_bytes(64, 3, 64) > 0
    assert lib.srwm_b200_srwm_reduce_scratch_bytes(4, 3, 7) == 0
    a = L.SrwmBwdArgs()
    a.N, a.H, a.L, a.E = 4, 2, 8, 16
    r = L.SrwmReduce()
    assert lib.srwm_b200_srwm_layer_backward_reduced(C.byref(a), None, None, None) == L.ERR_NULL
    assert lib.srwm_b200_srwm_layer_backward_reduced(C.byref(a), None, C.byref(r), None) == L.ERR_NULL   # no scratch
    r.scratch, r.scratch_bytes = 256, 16
    assert lib.srwm_b200_srwm_layer_backward_reduced(C.byref(a), None, C.byref(r), None) == L.ERR_TOO_LARGE
    r.scratch = 264
    assert lib.srwm_b200_srwm_layer_backward_reduced(C.byref(a), None, C.byref(r), None) == L.ERR_ALIGN


def _lanes_per_sequence_forward_id(E):
    """Id of the forward configuration that gives a sequence E lanes of a warp (srwm_fwd_warp_kernel),
    or None when this build of the library does not hold it for that head size."""
    from srwm_b200 import _lib as L
    for v in range(1, L.load().srwm_b200_num_variants(L.OP_SRWM_FWD, E)):
        d = L.describe(L.OP_SRWM_FWD, E, variant=v)
        if d["P"] == E and d["R"] == E:
            return v
    return None


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["plain", "softmax_shift", "softmax_shift_done"])
@pytest.mark.parametrize("E,N", [(E_, N_) for E_, N_ in [(32, 3), (16, 3), (16, 4), (8, 5)]
                                 if _lanes_per_sequence_forward_id(E_) is not None])   # head sizes this build holds it for
def test_lanes_per_sequence_forward_layer_level_form(E, N, mode, dt):
    """The forward that gives a sequence E lanes of a warp (one sequence per warp at d_head 32, two at 16,
    four at 8; the library's choice at d_head 32 on large grids).  Its layer-level form (input softmax,
    base + shift state, episode resets) is checked here on a small grid -- including sequence counts that
    leave part of the last warp without a sequence -- by asking for that configuration explicitly, against
    the default small-grid kernel (which the tests above hold to the oracle): outputs, final shift and
    every saved tensor."""
    from srwm_b200 import layer_ops as lo
    vid = _lanes_per_sequence_forward_id(E)
    d = torch.device("cuda", 0)
    H, L_ = 3, 37
    g = torch.Generator().manual_seed(77 + E + N)
    x = torch.randn(N, H, L_, E, generator=g).to(d, dt)
    std = E ** -0.5
    base = [(torch.randn(1, H, E, w, generator=g) * std).to(d) for w in (E, E, E, 4)]
    shift = done = None
    smx = False
    if mode != "plain":
        smx = True
        shift = [(0.1 * std * torch.randn(N, H, E, w, generator=g)).to(d) for w in (E, E, E, 4)]
    if mode == "softmax_shift_done":
        done = (torch.rand(N, L_, generator=g) < 0.2).to(d)
    ref = lo.srwm_layer_forward(x, base, shift, done, smx, variant=1)
    got = lo.srwm_layer_forward(x, base, shift, done, smx, variant=vid)
    tol = 8e-3 if dt == torch.bfloat16 else 1e-5
    assert orc.rel_max(got[0].float().cpu(), ref[0].float().cpu()) < tol
    for a, b in zip(got[1], ref[1]):
        assert float((a - b).abs().max()) < 1e-5 * std
    for a, b in zip(got[2], ref[2]):
        assert orc.rel_max(a.cpu(), b.cpu()) < 1e-5
    # without saving (inference): same output
    got2 = lo.srwm_layer_forward(x, base, shift, done, smx, save=False, variant=vid)
    assert torch.equal(got2[0], got[0]) and got2[2] is None
