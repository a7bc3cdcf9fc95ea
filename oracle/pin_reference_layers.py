"""Pin the layer-level oracle against the reference's own LAYER code and write golden fixtures.

TEST INFRASTRUCTURE.  Runs only in a checkout that has the upstream project next to it (pass
its root with ``--reference``); nothing else in this repository reads that tree.

The reference's layers (``supervised_learning/layer.py``, ``reinforcement_learning/torchbeast/
layer.py``) import CUDA-only operator packages.  Here those packages are loaded on the CPU the
same way ``pin_reference_main.py`` does it -- ``torch.utils.cpp_extension.load`` returns a
stand-in extension built on the pinned ``srwm_oracle.*_explicit`` functions, and the Function
classes' device dispatch tables get a "cpu" entry -- so the reference's own
``torch.autograd.Function`` classes and its own layer classes run unchanged, in float64.
The agents' layer file also imports operator packages that are not on this path
(``fast_transformers``, ``rec_update_fwm_tanh``, ``fast_weight_rnn_v2``, ``self_ref_v1``);
they are replaced by empty stand-ins (none of the layers exercised here uses them).

Cases (seeded inputs; every tensor of each run is stored under ``tests/golden/``):

* ``layer_sl_srwm``           ``SRWMlayer`` (supervised_learning/layer.py:112-209), input softmax on,
                              layer norm on, no state
* ``layer_sl_srwm_stateful``  the same layer, ``stateful=True``, with a carried state and
                              ``get_state=True`` (the loss reads the output only, see the note in the code)
* ``layer_sl_fastff``         ``FastFFlayer`` (supervised_learning/layer.py:49-108)
* ``layer_rl_sr_unroll``      ``SRlayer`` (reinforcement_learning/torchbeast/layer.py:340-421) driven
                              by the learner's loop (torchbeast_procgen/model.py:1180-1197):
                              ``state * notdone`` before every one-step call
* ``layer_rl_fastff``         the agents' ``FastFFlayer`` (torchbeast/layer.py:127-189) with a carried state

The CPU tests check ``srwm_layer_oracle`` against these fixtures (that is the pin of the layer
oracle); the GPU tests load the stored ``state_dict`` into this repository's layer modules and
check the fused kernels against them.

Usage:  python oracle/pin_reference_layers.py --reference /path/to/modern-srwm
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import pin_reference_main as prm  # noqa: E402  (stand-in extension functions)


def _load_operator_package(path, name, class_names):
    """Execute a reference operator package (its part above the self test) as module ``name``
    on the CPU and register the Function classes' callables under the "cpu" device key."""
    with open(path) as fh:
        src = fh.read()
    marker = "if __name__ == '__main__':"
    if marker in src:
        src = src[:src.index(marker)]
    src = src.replace('is not "cpu"', '!= "cuda-required"')
    src += "".join(f"{c}.dot['cpu'] = {c}.dot['cuda']\n{c}.dot_backward['cpu'] = {c}.dot_backward['cuda']\n"
                   for c in class_names)
    import torch.utils.cpp_extension as cpp_ext
    real = cpp_ext.load
    cpp_ext.load = prm._fake_load
    mod = types.ModuleType(name)
    mod.__file__ = path
    try:
        exec(compile(src, path, "exec"), mod.__dict__)
    finally:
        cpp_ext.load = real
    return mod


def _load_layer_file(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _grads(module):
    return {k: p.grad.clone() for k, p in module.named_parameters() if p.grad is not None}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("MODERN_SRWM_REFERENCE",
                                                          os.path.join(HERE, "..", "..", "reference")))
    ap.add_argument("--out", default=os.path.join(HERE, "..", "tests", "golden"))
    args = ap.parse_args()
    os.makedirs(args.out, exist_ok=True)
    torch.set_default_dtype(torch.float64)
    sl = os.path.join(args.reference, "supervised_learning")
    rl = os.path.join(args.reference, "reinforcement_learning", "torchbeast")

    # ---- supervised-learning layers ------------------------------------------------------
    sys.modules["self_ref_v0"] = _load_operator_package(
        os.path.join(sl, "self_ref_v0", "__init__.py"), "self_ref_v0", ["SelfRefv0", "StatefulSelfRefv0"])
    sys.modules["fast_weight"] = _load_operator_package(
        os.path.join(sl, "fast_weight", "__init__.py"), "fast_weight", ["DeltaFastWeight"])
    L_sl = _load_layer_file(os.path.join(sl, "layer.py"), "ref_sl_layer")

    H, E, D, T, B = 4, 16, 64, 21, 3
    g = torch.Generator().manual_seed(2024)

    def rn(*shape, scale=1.0):
        return torch.randn(*shape, generator=g) * scale

    torch.manual_seed(11)
    layer = L_sl.SRWMlayer(H, E, D, 0.0, use_ln=True, use_input_softmax=True, beta_init=-1.0, stateful=False)
    h = rn(T, B, D).requires_grad_()
    tgt = rn(T, B, D)
    out = layer(h)
    (out * tgt).sum().backward()
    torch.save(dict(cfg=dict(num_head=H, dim_head=E, in_dim=D, use_ln=True, use_input_softmax=True, stateful=False),
                    state_dict=layer.state_dict(), h=h.detach(), tgt=tgt, out=out.detach(), grad_h=h.grad,
                    grads=_grads(layer)), os.path.join(args.out, "layer_sl_srwm.pt"))

    torch.manual_seed(12)
    layer = L_sl.SRWMlayer(H, E, D, 0.0, use_ln=False, use_input_softmax=False, beta_init=-1.0, stateful=True)
    h = rn(T, B, D).requires_grad_()
    tgt = rn(T, B, D)
    state = [rn(B, H, E, E, scale=0.02).requires_grad_() for _ in range(3)] + [rn(B, H, E, 4, scale=0.02).requires_grad_()]
    out, new_state = layer(h, state=tuple(state), get_state=True)
    # The loss reads the output only.  A gradient flowing INTO the returned state is not pinned here:
    # the reference's stateful backward hands the incoming state gradients to its kernel as the
    # accumulators (self_ref_v0/__init__.py:182-210) and so does not return dL/dW_0 for them; that
    # path is checked against the autograd loop of srwm_oracle instead.
    (out * tgt).sum().backward()
    torch.save(dict(cfg=dict(num_head=H, dim_head=E, in_dim=D, use_ln=False, use_input_softmax=False, stateful=True),
                    state_dict=layer.state_dict(), h=h.detach(), tgt=tgt, state=[s.detach() for s in state],
                    out=out.detach(), new_state=[s.detach() for s in new_state], grad_h=h.grad,
                    grad_state=[s.grad for s in state], grads=_grads(layer)),
               os.path.join(args.out, "layer_sl_srwm_stateful.pt"))

    torch.manual_seed(13)
    Hd, Ed, Dd = 2, 32, 64
    layer = L_sl.FastFFlayer(Hd, Ed, Dd, 0.0)
    x = rn(T, B, Dd).requires_grad_()
    tgt = rn(T, B, Dd)
    out = layer(x)
    (out * tgt).sum().backward()
    torch.save(dict(cfg=dict(num_head=Hd, dim_head=Ed, in_dim=Dd), state_dict=layer.state_dict(), x=x.detach(),
                    tgt=tgt, out=out.detach(), grad_x=x.grad, grads=_grads(layer)),
               os.path.join(args.out, "layer_sl_fastff.pt"))

    # ---- the agents' layers -----------------------------------------------------------------
    tb = types.ModuleType("torchbeast")
    tb.__path__ = []
    sys.modules["torchbeast"] = tb
    sys.modules["torchbeast.self_ref_v0"] = _load_operator_package(
        os.path.join(rl, "self_ref_v0", "__init__.py"), "torchbeast.self_ref_v0", ["SelfRefv0"])
    sys.modules["torchbeast.fast_weight"] = _load_operator_package(
        os.path.join(rl, "fast_weight", "__init__.py"), "torchbeast.fast_weight", ["DeltaFastWeight"])
    for name, attr in (("fast_transformers", "fast_weight_sum"), ("rec_update_fwm_tanh", "rec_update_fwm_tanh"),
                       ("fast_weight_rnn_v2", "fast_rnn_v2"), ("self_ref_v1", "self_ref_v1")):
        m = types.ModuleType("torchbeast." + name)      # operators that are not on this path
        setattr(m, attr, None)
        sys.modules["torchbeast." + name] = m
    L_rl = _load_layer_file(os.path.join(rl, "layer.py"), "ref_rl_layer")

    torch.manual_seed(14)
    Hr, Er, Dr, Tr, Br = 4, 16, 64, 17, 4
    layer = L_rl.SRlayer(Hr, Er, Dr, 0.0)
    obs = rn(Tr, Br, Dr).requires_grad_()
    tgt = rn(Tr, Br, Dr)
    done = torch.rand(Tr, Br, generator=g) < 0.15
    done[0, 1] = True
    state0 = [rn(Br, Hr, Er, Er, scale=0.02) for _ in range(3)] + [rn(Br, Hr, Er, 4, scale=0.02)]
    state = tuple(state0)
    outs = []
    notdone = (~done).to(obs.dtype)
    for inp, nd in zip(obs.unbind(), notdone.unbind()):     # the loop of torchbeast_procgen/model.py:1180-1197
        nd = nd.view(-1, 1, 1, 1)
        state = tuple(nd * s for s in state)
        o, state = layer(inp.unsqueeze(0), state)
        outs.append(o)
    out = torch.cat(outs, 0)
    (out * tgt).sum().backward()
    torch.save(dict(cfg=dict(num_head=Hr, dim_head=Er, in_dim=Dr), state_dict=layer.state_dict(), obs=obs.detach(),
                    tgt=tgt, done=done, state0=state0, out=out.detach(), final_state=[s.detach() for s in state],
                    grad_obs=obs.grad, grads=_grads(layer)), os.path.join(args.out, "layer_rl_sr_unroll.pt"))

    torch.manual_seed(15)
    layer = L_rl.FastFFlayer(Hd, Ed, Dd, 0.0)
    x = rn(T, B, Dd).requires_grad_()
    tgt = rn(T, B, Dd)
    st = rn(B, Hd, Ed, Ed, scale=0.05)
    out, new_st = layer(x, state=st.clone())
    (out * tgt).sum().backward()
    torch.save(dict(cfg=dict(num_head=Hd, dim_head=Ed, in_dim=Dd), state_dict=layer.state_dict(), x=x.detach(),
                    tgt=tgt, state=st, out=out.detach(), new_state=new_st.detach(), grad_x=x.grad, grads=_grads(layer)),
               os.path.join(args.out, "layer_rl_fastff.pt"))
    print("wrote layer fixtures to", os.path.abspath(args.out))


if __name__ == "__main__":
    main()
