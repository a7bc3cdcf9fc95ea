"""CPU tests of the oracle: against the reference's own self-test tensors (golden
fixtures written by oracle/pin_reference_main.py) and against torch.autograd."""
import os

import pytest
import torch

import srwm_oracle as orc
from conftest import GOLDEN, delta_inputs, srwm_inputs


def _gold(name):
    return torch.load(os.path.join(GOLDEN, name))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-3), (torch.float64, 1e-3)])
def test_srwm_loop_matches_reference_main(dtype, tol):
    g = _gold("srwm_main_3x5x11x8.pt")
    x = g["x"].to(dtype).requires_grad_()
    Ws = [g[k].to(dtype).requires_grad_() for k in ("W_y", "W_q", "W_k", "w_b")]
    out, _ = orc.srwm_loop(x, *Ws)
    # the reference's own acceptance metric and threshold (self_ref_v0/__init__.py:229-233)
    assert orc.max_relative_error(out.detach().float(), g["out"]) < tol
    assert orc.rel_max(out.detach(), g["out"]) < 1e-5
    grads = torch.autograd.grad((out * g["grad_out"].to(dtype)).sum(), [x] + Ws)
    for got, key in zip(grads, ("grad_x", "grad_W_y", "grad_W_q", "grad_W_k", "grad_w_b")):
        assert orc.max_relative_error(got.float(), g[key]) < tol, key
        assert orc.rel_max(got, g[key]) < 2e-5, key


def test_srwm_explicit_matches_reference_main():
    g = _gold("srwm_main_3x5x11x8.pt")
    f = orc.srwm_forward_explicit(g["x"], g["W_y"], g["W_q"], g["W_k"], g["w_b"])
    assert orc.max_relative_error(f["out"], g["out"]) < 1e-3
    r = orc.srwm_backward_explicit(g["x"], f["q"], f["k"], f["beta"], f["y_diff"], f["q_diff"],
                                   f["k_diff"], f["beta_diff"], g["grad_out"], f["W_y"], f["W_q"],
                                   f["W_k"], f["w_b"])
    for got, key in zip(r[:5], ("grad_x", "grad_W_y", "grad_W_q", "grad_W_k", "grad_w_b")):
        assert orc.max_relative_error(got, g[key]) < 1e-3, key
    # the reversal lands back on the initial state
    for got, key in zip(r[5], ("W_y", "W_q", "W_k", "w_b")):
        assert orc.rel_max(got, g[key]) < 1e-5, key


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_delta_loop_matches_reference_main(dtype):
    g = _gold("delta_main_3x5x11x64.pt")
    Q, K, V, B = (g[k].to(dtype).requires_grad_() for k in ("Q", "K", "V", "beta"))
    W0 = torch.zeros(3, 5, 64, 64, dtype=dtype)
    out, _ = orc.delta_loop(Q, K, V, B, W0)
    assert orc.max_relative_error(out.detach().float(), g["out"]) < 1e-3
    grads = torch.autograd.grad((out * g["grad_out"].to(dtype)).sum(), [Q, K, V, B])
    for got, key in zip(grads, ("grad_Q", "grad_K", "grad_V", "grad_beta")):
        assert orc.max_relative_error(got.float(), g[key]) < 1e-3, key


def test_delta_explicit_matches_reference_main():
    g = _gold("delta_main_3x5x11x64.pt")
    W0 = torch.zeros(3, 5, 64, 64)
    f = orc.delta_forward_explicit(g["Q"], g["K"], g["V"], g["beta"], W0)
    assert orc.max_relative_error(f["out"], g["out"]) < 1e-3
    r = orc.delta_backward_explicit(g["Q"], g["K"], g["V"], g["beta"], f["v_old"], f["v_insert"],
                                    g["grad_out"], f["W"])
    for got, key in zip(r[:4], ("grad_Q", "grad_K", "grad_V", "grad_beta")):
        assert orc.max_relative_error(got, g[key]) < 1e-3, key
    assert float(r[4].abs().max()) < 1e-5    # W_0 = 0 rebuilt


@pytest.mark.parametrize("shape", [(2, 3, 9, 8), (1, 2, 1, 16), (2, 2, 17, 32)])
def test_srwm_explicit_equals_autograd_fp64(shape):
    N, H, L, E = shape
    x, Ws, go = srwm_inputs(N, H, L, E, seed=5)
    x = x.double().requires_grad_()
    Ws = [w.double().requires_grad_() for w in Ws]
    go = go.double()
    out, Wf = orc.srwm_loop(x, *Ws)
    gs = [torch.randn_like(w) for w in Wf]
    loss = (out * go).sum() + sum((w * g).sum() for w, g in zip(Wf, gs))
    want = torch.autograd.grad(loss, [x] + Ws)
    f = orc.srwm_forward_explicit(x.detach(), *[w.detach() for w in Ws])
    assert orc.rel_max(f["out"], out.detach()) < 1e-12
    r = orc.srwm_backward_explicit(x.detach(), f["q"], f["k"], f["beta"], f["y_diff"], f["q_diff"],
                                   f["k_diff"], f["beta_diff"], go, f["W_y"], f["W_q"], f["W_k"],
                                   f["w_b"], grad_state=gs)
    for got, w in zip(r[:5], want):
        assert orc.rel_max(got, w) < 1e-10
    for got, w in zip(r[5], Ws):
        assert orc.rel_max(got, w.detach()) < 1e-12


@pytest.mark.parametrize("shape", [(2, 3, 9, 8), (1, 2, 1, 16), (2, 2, 17, 64)])
def test_delta_explicit_equals_autograd_fp64(shape):
    N, H, L, E = shape
    Q, K, V, B, W0, go = (t.double() for t in delta_inputs(N, H, L, E, seed=6, w0="rand"))
    leaves = [t.requires_grad_() for t in (Q, K, V, B, W0)]
    out, WL = orc.delta_loop(*leaves)
    want = torch.autograd.grad((out * go).sum(), leaves)
    d = [t.detach() for t in leaves]
    f = orc.delta_forward_explicit(*d)
    assert orc.rel_max(f["out"], out.detach()) < 1e-12
    r = orc.delta_backward_explicit(d[0], d[1], d[2], d[3], f["v_old"], f["v_insert"], go, f["W"])
    for got, w in zip(r[:4] + (r[5],), want):
        assert orc.rel_max(got, w) < 1e-10
    assert orc.rel_max(r[4], d[4]) < 1e-12


def test_reference_loop_skips_last_update_without_changing_outputs():
    x, Ws, _ = srwm_inputs(2, 2, 6, 8, seed=9)
    a, Wa = orc.srwm_loop(x, *Ws, update_last=True)
    b, Wb = orc.srwm_loop(x, *Ws, update_last=False)
    assert torch.equal(a, b)
    assert not torch.equal(Wa[0], Wb[0])
