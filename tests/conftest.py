"""pytest configuration: the ``gpu`` marker, import paths, shared input generators."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "modern-srwm_b200"), os.path.join(ROOT, "oracle"), ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """Build the shared library if it is not there yet (nvcc cross-compiles without a GPU)."""
    lib = os.path.join(ROOT, "modern-srwm_b200", "srwm_b200", "libsrwm_b200.so")
    if not os.path.exists(lib):
        sys.path.insert(0, os.path.join(ROOT, "modern-srwm_b200", "csrc"))
        import build as _build
        _build.build()
    yield


def srwm_inputs(N, H, L, E, seed, weight="normal"):
    """Seeded SRWM inputs on the CPU in fp32.  weight='normal': N(0, 1/E) as the layer
    initialises them (supervised_learning/layer.py:148-154); 'uniform': U(-1,1) as the
    reference self test (supervised_learning/self_ref_v0/__init__.py:244-251)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, H, L, E, generator=g)
    if weight == "normal":
        std = E ** -0.5
        Ws = [torch.randn(N, H, E, E, generator=g) * std for _ in range(3)]
        Ws.append(torch.randn(N, H, E, 4, generator=g) * std)
    else:
        Ws = [torch.rand(N, H, E, E, generator=g) * 2 - 1 for _ in range(3)]
        Ws.append(torch.rand(N, H, E, 4, generator=g) * 2 - 1)
    go = torch.randn(N, H, L, E, generator=g)
    return x, Ws, go


def delta_inputs(N, H, L, E, seed, w0="zero"):
    """Seeded delta-rule inputs: q,k = softmax(N(0,1)), v ~ N(0,1), beta = sigmoid(N(0,1))."""
    g = torch.Generator().manual_seed(seed)
    Q = torch.softmax(torch.randn(N, H, L, E, generator=g), -1)
    K = torch.softmax(torch.randn(N, H, L, E, generator=g), -1)
    V = torch.randn(N, H, L, E, generator=g)
    B = torch.sigmoid(torch.randn(N, H, L, 1, generator=g))
    go = torch.randn(N, H, L, E, generator=g)
    W0 = torch.zeros(N, H, E, E) if w0 == "zero" else torch.randn(N, H, E, E, generator=g) * 0.1
    return Q, K, V, B, W0, go
