"""Drop-in hook: make the reference's own import statements resolve to this library,
with the reference tree left untouched.

    import srwm_b200.dropin          # installs the hook (idempotent)
    import layer                     # supervised_learning/layer.py, unchanged
    from torchbeast import layer     # reinforcement_learning/torchbeast/layer.py, unchanged

The reference imports its operators by package name:

    supervised_learning/layer.py:8-9
        from fast_weight import fast_weight_delta
        from self_ref_v0 import self_ref_v0, stateful_self_ref_v0
    reinforcement_learning/torchbeast/layer.py:7,11
        from torchbeast.fast_weight import fast_weight_delta
        from torchbeast.self_ref_v0 import self_ref_v0

and each of those packages compiles its ``.cu`` file at import time
(``torch.utils.cpp_extension.load``, self_ref_v0/__init__.py:19-27).  The import system
looks in ``sys.modules`` before it searches any path, so registering modules under those
four names is enough: the reference's packages are never executed, nothing is compiled at
import, and the names the layers use come from :mod:`srwm_b200.ops`.

The agents' ``layer.py`` also imports four operator packages that are not on this path
(``torchbeast.fast_transformers``, ``torchbeast.rec_update_fwm_tanh``,
``torchbeast.fast_weight_rnn_v2``, ``torchbeast.self_ref_v1``; layer.py:8-12).  By default they
are left alone (they build themselves as upstream does).  ``install(stub_other_operators=True)``
registers stand-ins for them whose functions raise when called, so that the file imports
without any JIT build; the SRWM and delta-rule layers never call them.
"""
from __future__ import annotations

import sys
import types

from . import ops

_OURS = {
    "self_ref_v0": ("SelfRefv0", "StatefulSelfRefv0", "self_ref_v0", "stateful_self_ref_v0"),
    "fast_weight": ("DeltaFastWeight", "fast_weight_delta"),
}
# operator packages of the agents' tree that this library does not replace: name -> exported functions
_OTHERS = {
    "fast_transformers": ("fast_weight_sum",),
    "rec_update_fwm_tanh": ("rec_update_fwm_tanh",),
    "fast_weight_rnn_v2": ("fast_rnn_v2",),
    "self_ref_v1": ("self_ref_v1",),
}
_installed = {}


def _module(name, attrs):
    m = types.ModuleType(name)
    m.__doc__ = f"srwm_b200 drop-in for the reference package `{name}`"
    m.__file__ = __file__
    m.__srwm_b200_dropin__ = True
    for a in attrs:
        setattr(m, a, getattr(ops, a))
    m.__all__ = list(attrs)
    return m


def _stub(name, fns):
    m = types.ModuleType(name)
    m.__doc__ = f"stand-in for `{name}` (not replaced by srwm_b200; raises when used)"
    m.__file__ = __file__
    m.__srwm_b200_dropin__ = True

    def make(fn):
        def raiser(*_a, **_k):
            raise NotImplementedError(
                f"{name}.{fn} is outside the path srwm_b200 replaces; install the hook with "
                "stub_other_operators=False to let the reference build its own extension")
        raiser.__name__ = fn
        return raiser

    for fn in fns:
        setattr(m, fn, make(fn))
    m.__all__ = list(fns)
    return m


def install(stub_other_operators=False, force=False):
    """Register the drop-in modules.  An operator package that is already imported from
    somewhere else is left in place unless ``force`` is given (and then replaced).  Returns
    the list of module names that now resolve to this library."""
    done = []
    for pkg, attrs in _OURS.items():
        for name in (pkg, "torchbeast." + pkg):
            cur = sys.modules.get(name)
            if cur is not None and not getattr(cur, "__srwm_b200_dropin__", False) and not force:
                # the sibling drop-in packages of this repository export the same objects
                if all(getattr(cur, a, None) is getattr(ops, a) for a in attrs):
                    done.append(name)
                continue
            m = _module(name, attrs)
            sys.modules[name] = m
            _installed[name] = m
            done.append(name)
    if stub_other_operators:
        for pkg, fns in _OTHERS.items():
            name = "torchbeast." + pkg
            if name not in sys.modules or force:
                m = _stub(name, fns)
                sys.modules[name] = m
                _installed[name] = m
    # a parent package imported later picks the submodules up from sys.modules; one that is
    # already imported gets them as attributes too
    tb = sys.modules.get("torchbeast")
    if tb is not None:
        for name, m in _installed.items():
            if name.startswith("torchbeast."):
                setattr(tb, name.split(".", 1)[1], m)
    return done


def uninstall():
    """Remove what :func:`install` registered."""
    for name, m in list(_installed.items()):
        if sys.modules.get(name) is m:
            del sys.modules[name]
        del _installed[name]


install()
