"""The import hook that lets the reference's layer files run over this library unchanged
(no GPU needed: only name resolution is checked here)."""
import importlib
import sys


def test_reference_import_lines_resolve_to_this_library():
    import srwm_b200.dropin as dropin
    import srwm_b200.ops as ops
    names = dropin.install(stub_other_operators=True)
    assert {"self_ref_v0", "fast_weight", "torchbeast.self_ref_v0", "torchbeast.fast_weight"} <= set(names)
    # supervised_learning/layer.py:8-9
    from fast_weight import fast_weight_delta
    from self_ref_v0 import self_ref_v0, stateful_self_ref_v0
    assert fast_weight_delta is ops.fast_weight_delta
    assert self_ref_v0 is ops.self_ref_v0 and stateful_self_ref_v0 is ops.stateful_self_ref_v0
    # reinforcement_learning/torchbeast/layer.py:7,11 -- no `torchbeast` package has to exist
    m1 = importlib.import_module("torchbeast.fast_weight")
    m2 = importlib.import_module("torchbeast.self_ref_v0")
    assert m1.fast_weight_delta is ops.fast_weight_delta and m2.self_ref_v0 is ops.self_ref_v0
    # the operator packages outside this path import as stand-ins that refuse to run
    m3 = importlib.import_module("torchbeast.self_ref_v1")
    try:
        m3.self_ref_v1()
    except NotImplementedError:
        pass
    else:
        raise AssertionError("stand-in operator ran")


def test_uninstall_removes_only_the_hook_modules():
    import srwm_b200.dropin as dropin
    dropin.install(stub_other_operators=True, force=True)
    dropin.uninstall()
    assert "torchbeast.self_ref_v1" not in sys.modules and "torchbeast.self_ref_v0" not in sys.modules
    dropin.install()
    assert "torchbeast.self_ref_v0" in sys.modules
