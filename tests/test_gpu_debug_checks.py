"""The debug build of the library (row checks that report through a status word instead of
faulting) on the GPU: the reporting path works, and the kernels raise no violation on sequence
lengths around their time-chunk length, on empty sequences and on strided views.

Runs in a child process because the build is chosen when the library is loaded
(``SRWM_B200_DEBUG=1``)."""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

CHILD = r'''
import sys, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[2])
import srwm_b200 as sb
from srwm_b200 import _lib as L
from srwm_b200 import layer_ops as lo
from conftest import srwm_inputs, delta_inputs
assert L.DEBUG_BUILD and L.LIB_PATH.endswith("libsrwm_b200_debug.so")
dev = torch.device("cuda", 0)
torch.cuda.set_device(dev)
ok, w = L.debug_status()
assert ok and w == 0, (ok, w)
# the reporting path: a check that must fail (no memory is touched by it)
L.check(L.load().srwm_b200_debug_selftest(None), "selftest")
ok, w = L.debug_status()
assert ok and (w >> 63) == 1 and ((w >> 48) & 0xff) == 255, hex(w)
assert L.debug_status() == (True, 0)            # cleared by the read
for E in (8, 16, 32, 64):
    for Ln in (0, 1, 15, 16, 17, 33):
        x, Ws, go = srwm_inputs(2, 3, Ln, E, 5)
        for dt in (torch.float32, torch.bfloat16):
            xd = x.permute(2, 0, 1, 3).contiguous().to(dev, dt).permute(1, 2, 0, 3)
            god = go.to(dev, dt)
            Wd = [t.to(dev) for t in Ws]
            out, saved = sb.srwm_forward(xd, *Wd)
            sb.srwm_backward(xd, saved, god, *Wd, restore_state=True)
            base = [t[:1].contiguous() for t in Wd]
            o2, sh, sv = lo.srwm_layer_forward(xd, base, None, None, True)
            if Ln > 0:
                lo.srwm_layer_backward(xd, sv, god, base, sh, None, True)
                lo.srwm_backward_detached(xd, sv, god, base[0], None, None, True)
        Q, K, V, B, W0, go = delta_inputs(2, 3, Ln, E, 6, "rand")
        for dt in (torch.float32, torch.bfloat16):
            Qd, Kd, Vd, Bd, god = (t.to(dev, dt) for t in (Q, K, V, B, go))
            W = W0.to(dev)
            out, saved = sb.delta_forward(Qd, Kd, Vd, Bd, W)
            sb.delta_backward(Qd, Kd, Vd, Bd, saved, god, W)
torch.cuda.synchronize()
ok, w = L.debug_status()
assert ok and w == 0, hex(w)
print("debug-build checks clean")
'''


def test_debug_build_reports_and_stays_clean():
    lib = os.path.join(ROOT, "modern-srwm_b200", "srwm_b200", "libsrwm_b200_debug.so")
    if not os.path.exists(lib):
        sys.path.insert(0, os.path.join(ROOT, "modern-srwm_b200", "csrc"))
        import build as _build
        _build.build(debug=True)
    env = dict(os.environ, SRWM_B200_DEBUG="1")
    r = subprocess.run([sys.executable, "-c", CHILD, os.path.join(ROOT, "modern-srwm_b200"), os.path.join(ROOT, "tests")],
                       capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "debug-build checks clean" in r.stdout
