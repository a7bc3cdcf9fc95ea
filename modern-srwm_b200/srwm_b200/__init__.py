"""B200-native SRWM / delta-rule recurrence operators (sm_100a kernels behind a C ABI).

Put the directory that contains this package on ``sys.path`` (it plays the role of the
reference's ``supervised_learning/`` script directory); the sibling packages
``self_ref_v0`` and ``fast_weight`` then satisfy the reference's own imports
(``from self_ref_v0 import self_ref_v0, stateful_self_ref_v0``,
``from fast_weight import fast_weight_delta``; supervised_learning/layer.py:8-9).
"""
from .ops import (DeltaFastWeight, SelfRefv0, StatefulSelfRefv0, delta_backward, delta_forward,
                  fast_weight_delta, reduce_batch, self_ref_v0, set_variant, srwm_backward,
                  srwm_forward, stateful_self_ref_v0)

__all__ = ["self_ref_v0", "stateful_self_ref_v0", "fast_weight_delta", "SelfRefv0",
           "StatefulSelfRefv0", "DeltaFastWeight", "srwm_forward", "srwm_backward",
           "delta_forward", "delta_backward", "reduce_batch", "set_variant"]
