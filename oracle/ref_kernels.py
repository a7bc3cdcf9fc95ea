"""Loader and thin callers for the reference's own CUDA extensions built by
``oracle/build_ref_kernels.py`` into ``oracle/_ref/`` (TEST INFRASTRUCTURE).

``available()`` is False when the modules were not built (they cannot be built without the
upstream sources).  The callers allocate zero-filled outputs exactly as the reference's
autograd functions do (self_ref_v0/__init__.py:56-65, fast_weight/__init__.py:48-50),
because its kernels accumulate with atomicAdd.

Valid envelope of the reference kernels (read from their source): the SRWM backward indexes
its staged q/k rows with the wrong stride whenever d_head**2 > 768 and d_head does not tile
it (d_head 28..47 and 64), and neither SRWM kernel chains correctly over more than one
shared-memory time chunk in the backward; callers here must stay at d_head <= 16 and short
sequences for SRWM.  The delta kernels are valid for any L at d = 64.
"""
import importlib.util
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF = os.path.join(_HERE, "_ref")
_mods = {}


def _so(name):
    d = os.path.join(_REF, name)
    p = os.path.join(d, name + ".so")
    return p if os.path.exists(p) else None


def available():
    return _so("ref_self_ref") is not None and _so("ref_fast_weight") is not None


def _load(name):
    if name not in _mods:
        spec = importlib.util.spec_from_file_location(name, _so(name))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _mods[name] = mod
    return _mods[name]


def srwm_forward(x, W_y, W_q, W_k, w_b):
    """Reference forward; mutates W_* (final state).  Returns out and the saved tensors."""
    m = _load("ref_self_ref")
    N, H, L, E = x.shape
    z = lambda *s: torch.zeros(s, device=x.device, dtype=x.dtype)
    out, q, k, yd, qd, kd = (z(N, H, L, E) for _ in range(6))
    beta, bd = z(N, H, L, 4), z(N, H, L, 4)
    m.self_ref_forward(x, W_y, W_q, W_k, w_b, q, k, beta, yd, qd, kd, bd, out)
    return out, (q, k, beta, yd, qd, kd, bd)


def srwm_backward(x, saved, grad_out, W_y, W_q, W_k, w_b):
    m = _load("ref_self_ref")
    q, k, beta, yd, qd, kd, bd = saved
    gx = torch.zeros_like(x)
    gW = [torch.zeros_like(w) for w in (W_y, W_q, W_k, w_b)]
    m.self_ref_backward(x, q, k, beta, yd, qd, kd, bd, grad_out, W_y, W_q, W_k, w_b, gx, *gW)
    return (gx, *gW)


def delta_forward(Q, K, V, beta, W):
    m = _load("ref_fast_weight")
    N, H, L, E = Q.shape
    M = V.shape[-1]
    z = lambda: torch.zeros((N, H, L, M), device=Q.device, dtype=Q.dtype)
    out, v_old, v_ins = z(), z(), z()
    m.fast_weight_forward(Q, K, V, beta, v_old, v_ins, W, out)
    return out, (v_old, v_ins)


def delta_backward(Q, K, V, beta, saved, grad_out, W):
    m = _load("ref_fast_weight")
    v_old, v_ins = saved
    gQ, gK, gV, gB = (torch.zeros_like(t) for t in (Q, K, V, beta))
    m.fast_weight_backward(Q, K, V, beta, v_old, v_ins, grad_out, W, gQ, gK, gV, gB)
    return gQ, gK, gV, gB
