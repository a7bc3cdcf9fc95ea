"""GPU check against the reference's own CUDA kernels (built unmodified into oracle/_ref by
oracle/build_ref_kernels.py), inside their valid envelope: SRWM at d_head 8 and 16 with short
sequences, delta rule at d 64.  Skipped when the reference build is not present."""
import pytest
import torch

import srwm_oracle as orc
from conftest import delta_inputs, srwm_inputs

pytestmark = pytest.mark.gpu


def _ref():
    import ref_kernels
    if not ref_kernels.available():
        pytest.skip("oracle/_ref not built (needs the upstream sources)")
    return ref_kernels


@pytest.mark.parametrize("shape", [(3, 5, 11, 8), (4, 4, 64, 16)])
def test_srwm_matches_reference_cuda_kernels(shape):
    import srwm_b200 as sb
    ref = _ref()
    d = torch.device("cuda", 0)
    N, H, L, E = shape
    x, Ws, go = srwm_inputs(N, H, L, E, seed=101)
    xd, god = x.to(d), go.to(d)
    Wr = [w.to(d).clone() for w in Ws]
    out_r, saved_r = ref.srwm_forward(xd, *Wr)
    grads_r = ref.srwm_backward(xd, saved_r, god, *Wr)
    Wo = [w.to(d).clone() for w in Ws]
    out_o, saved_o = sb.srwm_forward(xd, *Wo)
    grads_o = sb.srwm_backward(xd, saved_o, god, *Wo)
    assert orc.rel_max(out_o, out_r) < 1e-4
    for a, b in zip(saved_o, saved_r):
        assert orc.rel_max(a, b) < 1e-4
    for a, b in zip(Wo, Wr):                      # final state left in place by both
        assert orc.rel_max(a, b) < 1e-4
    for a, b in zip(grads_o, grads_r):
        assert orc.rel_max(a, b) < 1e-3


def test_delta_matches_reference_cuda_kernels():
    import srwm_b200 as sb
    ref = _ref()
    d = torch.device("cuda", 0)
    Q, K, V, B, W0, go = (t.to(d) for t in delta_inputs(3, 5, 150, 64, seed=102))
    Wr = W0.clone()
    out_r, saved_r = ref.delta_forward(Q, K, V, B, Wr)
    WL_r = Wr.clone()
    grads_r = ref.delta_backward(Q, K, V, B, saved_r, go, Wr)
    Wo = W0.clone()
    out_o, saved_o = sb.delta_forward(Q, K, V, B, Wo)
    assert orc.rel_max(Wo, WL_r) < 1e-4
    grads_o = sb.delta_backward(Q, K, V, B, saved_o, go, Wo)
    assert orc.rel_max(out_o, out_r) < 1e-4
    for a, b in zip(saved_o, saved_r):
        assert orc.rel_max(a, b) < 1e-4
    for a, b in zip(grads_o[:4], grads_r):
        assert orc.rel_max(a, b) < 1e-3
    assert float((Wo - Wr).abs().max()) < 1e-5    # both restore W_0
