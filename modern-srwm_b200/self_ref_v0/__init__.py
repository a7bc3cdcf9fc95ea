"""Drop-in for the reference package ``self_ref_v0``
(supervised_learning/self_ref_v0/__init__.py; the torchbeast copy exports the same
``self_ref_v0`` name).  No JIT build happens at import: the kernels come from the
prebuilt libsrwm_b200.so."""
import os as _os
import sys as _sys

_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))
from srwm_b200.ops import SelfRefv0, StatefulSelfRefv0, self_ref_v0, stateful_self_ref_v0  # noqa: E402

__all__ = ["SelfRefv0", "StatefulSelfRefv0", "self_ref_v0", "stateful_self_ref_v0"]
