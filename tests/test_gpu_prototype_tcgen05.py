"""The tcgen05 prototype of the chunkwise delta-rule forward (modern-srwm_b200/csrc/prototype/): builds
the standalone program with nvcc and checks the errors it reports against its own CPU recurrence.
The saved v_insert and the final state are held to fp32-level bounds (W and U are split in two tf32
terms); out and v_old to the tf32 bound of the unsplit triangular factors."""
import os
import re
import shutil
import subprocess

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def test_chunkwise_tcgen05_prototype_runs_and_is_tf32_accurate(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    src = os.path.join(ROOT, "modern-srwm_b200", "csrc", "prototype", "delta_chunk_tcgen05.cu")
    exe = str(tmp_path / "delta_chunk_tcgen05")
    subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-o", exe, src])
    out = subprocess.run([exe, "6", "320"], capture_output=True, text=True, timeout=120, check=True).stdout
    assert "kernel: no error" in out, out
    m = re.search(r"status (\d+).*out (\S+)\s+v_old (\S+)\s+v_ins (\S+)\s+W_L (\S+)", out)
    assert m, out
    assert int(m.group(1)) == 0                      # no bounded wait gave up
    errs = [float(m.group(i)) for i in range(2, 6)]
    assert errs[0] < 2e-3 and errs[1] < 2e-3 and errs[2] < 1e-5 and errs[3] < 1e-4, out
