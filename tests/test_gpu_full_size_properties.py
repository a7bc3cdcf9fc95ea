"""The two largest configurations at their full size, checked through properties that do not need
the oracle to run at that size.

A launch over 16384 (SRWM) or 8192 (delta rule) sequences cannot be replayed by the CPU oracle, but
every (sample, head) sequence is independent of all the others and the forward is causal in time, so

* a sequence taken out of the big launch and run alone must give bit-identical results (same
  kernel, same arithmetic; any cross-talk between CTAs, wrong offset at large indices, or 32-bit
  overflow in the address arithmetic would show), and
* the first half of a sequence, run alone, must reproduce the first half of its outputs bit for bit.

One of the picked sequences is also compared with the float64 oracle, which ties the big launch to
the reference's arithmetic (supervised_learning/self_ref_v0/__init__.py:296-356,
supervised_learning/fast_weight/__init__.py:167-191).

Sizes: SRWM B=1024 H=16 L=2048 d=64 and delta rule B=512 H=16 L=8192 d=64, bf16 activations, fp32
state: about 65 GB and 105 GB on the device.  Skipped when the GPU has less free memory than that.
"""
import pytest
import torch

import srwm_oracle as orc

pytestmark = pytest.mark.gpu
BF16_TOL, GRAD_TOL = 8e-3, 1e-3


def _dev():
    return torch.device("cuda", 0)


def _need(gb):
    torch.cuda.empty_cache()
    free, _ = torch.cuda.mem_get_info(_dev())
    if free < gb * 2 ** 30:
        pytest.skip(f"needs {gb} GiB of free device memory, {free / 2 ** 30:.0f} available")


def _fill(shape, dt, gen, fn=None, step=32):
    """Random tensor built in slices over the batch so that the fp32 temporaries stay small."""
    out = torch.empty(shape, device=_dev(), dtype=dt)
    for n0 in range(0, shape[0], step):
        n1 = min(shape[0], n0 + step)
        t = torch.randn((n1 - n0, *shape[1:]), device=_dev(), generator=gen)
        out[n0:n1] = (fn(t) if fn else t).to(dt)
    return out


def _picks(B, H):
    # first and last CTA, and sequences in the middle of different waves
    return [(0, 0), (B - 1, H - 1), (B // 2, 5), (37, 11), (B // 3, 0), (701 % B, H - 1)]


def _take(t, picks):
    return torch.stack([t[n, h] for n, h in picks]).unsqueeze(1).contiguous()


def test_srwm_largest_configuration_sequences_are_independent_and_causal():
    import srwm_b200 as sb
    _need(80)
    d = _dev()
    B, H, L, E = 1024, 16, 2048, 64
    g = torch.Generator(device=d).manual_seed(1005)
    x = _fill((B, H, L, E), torch.bfloat16, g)
    go = _fill((B, H, L, E), torch.bfloat16, g)
    std = E ** -0.5
    slow = [torch.randn(1, H, E, w, device=d, generator=g) * std for w in (E, E, E, 4)]
    W = [w.repeat(B, 1, 1, 1) for w in slow]
    out, saved = sb.srwm_forward(x, *W, variant=0)
    grads = sb.srwm_backward(x, saved, go, *W, variant=0)
    torch.cuda.synchronize()

    picks = _picks(B, H)
    xs, gos = _take(x, picks), _take(go, picks)
    Ws = [torch.stack([w[0, h] for _, h in picks]).unsqueeze(1).contiguous() for w in slow]
    outs, saveds = sb.srwm_forward(xs, *Ws, variant=0)
    gradss = sb.srwm_backward(xs, saveds, gos, *Ws, variant=0)
    assert torch.equal(outs, _take(out, picks))
    for a, b in zip(saveds, saved):
        assert torch.equal(a, _take(b, picks))
    for a, b in zip(Ws, W):                      # final state
        assert torch.equal(a, _take(b, picks))
    for a, b in zip(gradss, grads):
        assert torch.equal(a, _take(b, picks))

    # causality of the forward: half the steps, same first half
    Wh = [torch.stack([w[0, h] for _, h in picks]).unsqueeze(1).contiguous() for w in slow]
    outh, savedh = sb.srwm_forward(xs[:, :, :L // 2].contiguous(), *Wh, variant=0)
    assert torch.equal(outh, outs[:, :, :L // 2])
    for a, b in zip(savedh, saveds):
        assert torch.equal(a, b[:, :, :L // 2])

    # one sequence of the big launch against the float64 oracle
    n, h = picks[2]
    x1 = x[n:n + 1, h:h + 1].cpu().double()
    go1 = go[n:n + 1, h:h + 1].cpu().double()
    W1 = [w[:, h:h + 1].cpu().double() for w in slow]
    f = orc.srwm_forward_explicit(x1, *W1)
    r = orc.srwm_backward_explicit(x1, f["q"], f["k"], f["beta"], f["y_diff"], f["q_diff"], f["k_diff"],
                                   f["beta_diff"], go1, f["W_y"], f["W_q"], f["W_k"], f["w_b"])
    assert orc.rel_max(out[n:n + 1, h:h + 1].float().cpu(), f["out"]) < BF16_TOL
    assert orc.rel_max(grads[0][n:n + 1, h:h + 1].float().cpu(), r[0]) < BF16_TOL
    for t, o in zip(grads[1:], r[1:5]):
        assert orc.rel_max(t[n:n + 1, h:h + 1].cpu(), o) < GRAD_TOL
    del x, go, out, saved, grads, W
    torch.cuda.empty_cache()


def test_delta_largest_configuration_sequences_are_independent_and_causal():
    import srwm_b200 as sb
    _need(125)
    d = _dev()
    B, H, L, E = 512, 16, 8192, 64
    g = torch.Generator(device=d).manual_seed(1006)
    sm = lambda t: torch.softmax(t, -1)
    Q = _fill((B, H, L, E), torch.bfloat16, g, sm, step=16)
    K = _fill((B, H, L, E), torch.bfloat16, g, sm, step=16)
    V = _fill((B, H, L, E), torch.bfloat16, g, None, step=16)
    Bt = _fill((B, H, L, 1), torch.bfloat16, g, torch.sigmoid)
    go = _fill((B, H, L, E), torch.bfloat16, g, None, step=16)
    W = torch.zeros(B, H, E, E, device=d)
    out, saved = sb.delta_forward(Q, K, V, Bt, W, variant=0)
    WL = W.clone()
    grads = sb.delta_backward(Q, K, V, Bt, saved, go, W, variant=0)
    torch.cuda.synchronize()
    # the backward walks the state back to W_0 = 0, up to the rounding of undoing 8192 updates
    assert float(W.abs().max()) <= 1e-3 * float(WL.abs().max())

    # the kernels that the automatic choice takes at 8192 sequences, by number, for the small launch
    picks = _picks(B, H)
    sub = lambda t: _take(t, picks)
    Qs, Ks, Vs, Bs, gos = sub(Q), sub(K), sub(V), sub(Bt), sub(go)
    Wz = torch.zeros(len(picks), 1, E, E, device=d)
    outs, saveds = sb.delta_forward(Qs, Ks, Vs, Bs, Wz, variant=1)
    assert torch.equal(outs, sub(out))
    for a, b in zip(saveds, saved):
        assert torch.equal(a, sub(b))
    assert torch.equal(Wz, sub(WL))
    gradss = sb.delta_backward(Qs, Ks, Vs, Bs, saveds, gos, Wz, variant=1)
    for a, b in zip(gradss[:4], grads[:4]):
        assert torch.equal(a, sub(b))

    Wh = torch.zeros(len(picks), 1, E, E, device=d)
    half = lambda t: t[:, :, :L // 2].contiguous()
    outh, savedh = sb.delta_forward(half(Qs), half(Ks), half(Vs), half(Bs), Wh, variant=1)
    assert torch.equal(outh, outs[:, :, :L // 2])
    for a, b in zip(savedh, saveds):
        assert torch.equal(a, b[:, :, :L // 2])

    n, h = picks[3]
    one = lambda t: t[n:n + 1, h:h + 1].float().cpu().double()
    W0 = torch.zeros(1, 1, E, E, dtype=torch.float64)
    f = orc.delta_forward_explicit(one(Q), one(K), one(V), one(Bt), W0)
    assert orc.rel_max(out[n:n + 1, h:h + 1].float().cpu(), f["out"]) < BF16_TOL
    r = orc.delta_backward_explicit(one(Q), one(K), one(V), one(Bt), f["v_old"], f["v_insert"], one(go), f["W"])
    for t, o in zip(grads[:4], r[:4]):
        assert orc.rel_max(t[n:n + 1, h:h + 1].float().cpu(), o) < BF16_TOL
    del Q, K, V, go, out, saved, grads, W, WL
    torch.cuda.empty_cache()
