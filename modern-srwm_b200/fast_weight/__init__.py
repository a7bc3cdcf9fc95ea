"""Drop-in for the reference package ``fast_weight``
(supervised_learning/fast_weight/__init__.py; the torchbeast copy exports the same
``fast_weight_delta`` name).  No JIT build happens at import: the kernels come from the
prebuilt libsrwm_b200.so."""
import os as _os
import sys as _sys

_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))
from srwm_b200.ops import DeltaFastWeight, fast_weight_delta  # noqa: E402

__all__ = ["DeltaFastWeight", "fast_weight_delta"]
