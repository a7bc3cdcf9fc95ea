"""The reference's own LAYER code as the pin: fixtures under tests/golden/layer_*.pt were produced by
oracle/pin_reference_layers.py, which runs the reference's layer classes (and their autograd
Functions) unchanged on the CPU in float64.

CPU part: the layer-level oracle (oracle/srwm_layer_oracle.py) reproduces those runs, which is
what pins it.  GPU part: this repository's layer modules, loaded with the stored state_dict,
reproduce them through the fused kernels (forward <= 1e-4, gradients <= 1e-3).
"""
import os

import pytest
import torch
import torch.nn.functional as F

import srwm_layer_oracle as lorc
import srwm_oracle as orc
from conftest import GOLDEN

FWD_TOL, GRAD_TOL = 1e-4, 1e-3


def _load(name):
    return torch.load(os.path.join(GOLDEN, name + ".pt"))


def _heads(h, H, E):
    L, B, _ = h.shape
    return h.reshape(L, B, H, E).permute(1, 2, 0, 3)


def _merge(o):
    B, H, L, E = o.shape
    return o.transpose(1, 2).reshape(B, L, H * E).transpose(0, 1)


def _p(g, names):
    return [g["state_dict"][n].clone().requires_grad_() for n in names]


# ---------------------------------------------------------------------------------------
# CPU: the layer oracle against the reference layers' runs
# ---------------------------------------------------------------------------------------

def test_oracle_matches_reference_srwm_layer():
    g = _load("layer_sl_srwm")
    c = g["cfg"]
    W = _p(g, ["W_y", "W_q", "W_k", "w_b"])
    ln_w, ln_b, wo = _p(g, ["layer_norm.weight", "layer_norm.bias", "out_linear.weight"])
    h = g["h"].clone().requires_grad_()
    o, _ = lorc.srwm_layer(_heads(h, c["num_head"], c["dim_head"]), W, None, input_softmax=True)
    out = F.layer_norm(h, (c["in_dim"],), ln_w, ln_b) + F.linear(_merge(o), wo)
    (out * g["tgt"]).sum().backward()
    assert orc.rel_max(out.detach(), g["out"]) < 1e-10
    assert orc.rel_max(h.grad, g["grad_h"]) < 1e-9
    for t, n in zip(W + [ln_w, ln_b, wo], ["W_y", "W_q", "W_k", "w_b", "layer_norm.weight", "layer_norm.bias",
                                            "out_linear.weight"]):
        assert orc.rel_max(t.grad, g["grads"][n]) < 1e-9, n


def test_oracle_matches_reference_stateful_srwm_layer():
    g = _load("layer_sl_srwm_stateful")
    c = g["cfg"]
    W = _p(g, ["W_y", "W_q", "W_k", "w_b"])
    (wo,) = _p(g, ["out_linear.weight"])
    h = g["h"].clone().requires_grad_()
    st = [s.clone().requires_grad_() for s in g["state"]]
    o, new = lorc.srwm_layer(_heads(h, c["num_head"], c["dim_head"]), W, st, input_softmax=False)
    out = h + F.linear(_merge(o), wo)
    (out * g["tgt"]).sum().backward()
    assert orc.rel_max(out.detach(), g["out"]) < 1e-10
    for a, b in zip(new, g["new_state"]):
        assert float((a.detach() - b).abs().max()) < 1e-10
    assert orc.rel_max(h.grad, g["grad_h"]) < 1e-9
    for a, b in zip(st, g["grad_state"]):
        assert orc.rel_max(a.grad, b) < 1e-9
    for t, n in zip(W + [wo], ["W_y", "W_q", "W_k", "w_b", "out_linear.weight"]):
        assert orc.rel_max(t.grad, g["grads"][n]) < 1e-9, n


def test_oracle_matches_reference_learner_unroll():
    g = _load("layer_rl_sr_unroll")
    c = g["cfg"]
    W = _p(g, ["W_y", "W_q", "W_k", "w_b"])
    (wo,) = _p(g, ["out_linear.weight"])
    obs = g["obs"].clone().requires_grad_()
    o, fin = lorc.srwm_unroll_detached(_heads(obs, c["num_head"], c["dim_head"]), W, g["state0"], g["done"].t(), True)
    out = obs + F.linear(_merge(o), wo)
    (out * g["tgt"]).sum().backward()
    assert orc.rel_max(out.detach(), g["out"]) < 1e-10
    for a, b in zip(fin, g["final_state"]):
        assert float((a - b).abs().max()) < 1e-10
    assert orc.rel_max(obs.grad, g["grad_obs"]) < 1e-9
    assert orc.rel_max(W[0].grad, g["grads"]["W_y"]) < 1e-9
    assert orc.rel_max(wo.grad, g["grads"]["out_linear.weight"]) < 1e-9
    for t, n in zip(W[1:], ["W_q", "W_k", "w_b"]):     # the detached state passes them nothing
        assert t.grad is None or float(t.grad.abs().max()) == 0.0
        assert n not in g["grads"] or float(g["grads"][n].abs().max()) == 0.0


@pytest.mark.parametrize("name,eps", [("layer_sl_fastff", 0.0), ("layer_rl_fastff", 1e-5)])
def test_oracle_matches_reference_delta_layers(name, eps):
    g = _load(name)
    c = g["cfg"]
    H, E = c["num_head"], c["dim_head"]
    ws, ln_w, ln_b, wo = _p(g, ["slow_net.weight", "layer_norm.weight", "layer_norm.bias", "out_linear.weight"])
    x = g["x"].clone().requires_grad_()
    L, B, _ = x.shape
    rows = F.linear(F.layer_norm(x, (c["in_dim"],), ln_w, ln_b), ws).view(L, B, H, 3 * E + 1).permute(1, 2, 0, 3)
    W0 = g["state"] if "state" in g else torch.zeros(B, H, E, E, dtype=x.dtype)
    o, WL = lorc.delta_layer(rows, W0, eps)
    out = x + F.linear(_merge(o), wo)
    (out * g["tgt"]).sum().backward()
    assert orc.rel_max(out.detach(), g["out"]) < 1e-10
    if "new_state" in g:
        assert orc.rel_max(WL.detach(), g["new_state"]) < 1e-10
    assert orc.rel_max(x.grad, g["grad_x"]) < 1e-9
    for t, n in zip([ws, ln_w, ln_b, wo], ["slow_net.weight", "layer_norm.weight", "layer_norm.bias", "out_linear.weight"]):
        assert orc.rel_max(t.grad, g["grads"][n]) < 1e-9, n


# ---------------------------------------------------------------------------------------
# GPU: this repository's layer modules against the same runs
# ---------------------------------------------------------------------------------------

def _module(cls, g, **kw):
    d = torch.device("cuda", 0)
    c = g["cfg"]
    m = cls(c["num_head"], c["dim_head"], c["in_dim"], 0.0, **kw)
    m.load_state_dict({k: v.float() for k, v in g["state_dict"].items()})
    return m.to(d), d


def _check_grads(m, g):
    for n, p in m.named_parameters():
        if n in g["grads"]:
            ref = g["grads"][n]
            if float(ref.abs().max()) == 0.0:
                assert p.grad is None or float(p.grad.abs().max()) == 0.0, n
            else:
                assert orc.rel_max(p.grad.cpu(), ref) < GRAD_TOL, n


@pytest.mark.gpu
def test_gpu_srwm_layer_reproduces_reference_layer():
    from srwm_b200.layers import SRWMlayer
    g = _load("layer_sl_srwm")
    m, d = _module(SRWMlayer, g, use_ln=True, use_input_softmax=True)
    h = g["h"].float().to(d).requires_grad_()
    out = m(h)
    (out * g["tgt"].float().to(d)).sum().backward()
    assert orc.rel_max(out.detach().cpu(), g["out"]) < FWD_TOL
    assert orc.rel_max(h.grad.cpu(), g["grad_h"]) < GRAD_TOL
    _check_grads(m, g)


@pytest.mark.gpu
def test_gpu_stateful_srwm_layer_reproduces_reference_layer():
    from srwm_b200.layers import SRWMlayer
    g = _load("layer_sl_srwm_stateful")
    m, d = _module(SRWMlayer, g, use_ln=False, use_input_softmax=False, stateful=True)
    h = g["h"].float().to(d).requires_grad_()
    st = [s.float().to(d).requires_grad_() for s in g["state"]]
    out, new = m(h, state=tuple(st), get_state=True)
    (out * g["tgt"].float().to(d)).sum().backward()
    assert orc.rel_max(out.detach().cpu(), g["out"]) < FWD_TOL
    scale = float(g["state_dict"]["W_y"].abs().max())
    for a, b in zip(new, g["new_state"]):
        assert float((a.detach().cpu() - b).abs().max()) < FWD_TOL * scale
    assert orc.rel_max(h.grad.cpu(), g["grad_h"]) < GRAD_TOL
    for a, b in zip(st, g["grad_state"]):
        assert orc.rel_max(a.grad.cpu(), b) < GRAD_TOL
    _check_grads(m, g)


@pytest.mark.gpu
def test_gpu_sr_layer_unroll_reproduces_reference_learner_loop():
    from srwm_b200.layers import SRlayer
    g = _load("layer_rl_sr_unroll")
    m, d = _module(SRlayer, g)
    obs = g["obs"].float().to(d).requires_grad_()
    out, fin = m.unroll(obs, g["done"].to(d), [s.float().to(d) for s in g["state0"]])
    (out * g["tgt"].float().to(d)).sum().backward()
    assert orc.rel_max(out.detach().cpu(), g["out"]) < FWD_TOL
    scale = float(g["state_dict"]["W_y"].abs().max())
    for a, b in zip(fin, g["final_state"]):
        assert float((a.cpu() - b).abs().max()) < FWD_TOL * scale
    assert orc.rel_max(obs.grad.cpu(), g["grad_obs"]) < GRAD_TOL
    _check_grads(m, g)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["layer_sl_fastff", "layer_rl_fastff"])
def test_gpu_fast_ff_layers_reproduce_reference_layers(name):
    from srwm_b200.layers import FastFFlayer, FastFFlayerRL
    g = _load(name)
    m, d = _module(FastFFlayerRL if "state" in g else FastFFlayer, g)
    x = g["x"].float().to(d).requires_grad_()
    if "state" in g:
        out, new = m(x, g["state"].float().to(d).clone())
        assert orc.rel_max(new.cpu(), g["new_state"]) < FWD_TOL
    else:
        out = m(x)
    (out * g["tgt"].float().to(d)).sum().backward()
    assert orc.rel_max(out.detach().cpu(), g["out"]) < FWD_TOL
    assert orc.rel_max(x.grad.cpu(), g["grad_x"]) < GRAD_TOL
    _check_grads(m, g)
