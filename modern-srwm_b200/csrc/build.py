"""Build libsrwm_b200.so in-tree for sm_100a with nvcc (no torch, no JIT).

    python modern-srwm_b200/csrc/build.py [--force] [--verbose] [--tuning]

Every kernel translation unit is compiled twice (fp32 and bf16 activation streams) and
the objects are linked, together with the C ABI, into
``modern-srwm_b200/srwm_b200/libsrwm_b200.so``.  nvcc cross-compiles, so this works on a
machine without a GPU.  Objects are rebuilt only when a source or header is newer (or the
flags changed).  ``--tuning`` also compiles the alternative kernel configurations of
``configs.h`` (explicit variant ids beyond the ones the library itself picks), for A/B timing.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

CSRC = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(CSRC)
ROOT = os.path.dirname(PKG)
INCLUDE = os.path.join(ROOT, "include")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(PKG, "srwm_b200", "libsrwm_b200.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I", INCLUDE, "-I", CSRC]
KERNEL_TUS = ["kernels_srwm_fwd", "kernels_srwm_bwd", "kernels_srwm_bwd_det", "kernels_delta_fwd",
              "kernels_delta_bwd"]


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(INCLUDE, "srwm_b200.h"))
    return hs


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(job):
    src, obj, extra, verbose = job
    cmd = [_nvcc()] + ARCH + COMMON + extra + ["-c", src, "-o", obj]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    return obj, r.returncode, r.stdout + r.stderr


def build(force=False, verbose=False, tuning=None, debug=False):
    if debug:   # a separate library with the row checks compiled in (objects in their own directory)
        return _build(os.path.join(CSRC, "build_debug"), os.path.join(PKG, "srwm_b200", "libsrwm_b200_debug.so"),
                      force, verbose, False, ["-DSRWM_DEBUG_CHECKS"])
    return _build(OBJ, LIB, force, verbose, tuning, [])


def _build(OBJ, LIB, force, verbose, tuning, extra_flags):
    os.makedirs(OBJ, exist_ok=True)
    hdrs = _headers()
    # the flag set the objects were built with; a change rebuilds everything.  tuning=None keeps
    # whatever the existing objects were built with (so that a plain rebuild does not flip it).
    stamp = os.path.join(OBJ, "flags.txt")
    prev = open(stamp).read().strip() if os.path.exists(stamp) else ""
    if tuning is None:
        tuning = prev == "tuning"
    cur = "tuning" if tuning else "product"
    if cur != prev:
        force = True
    extra_all = (["-DSRWM_TUNING_VARIANTS"] if tuning else []) + list(extra_flags)
    jobs = []
    for tu in KERNEL_TUS:
        src = os.path.join(CSRC, tu + ".cu")
        for bf in (0, 1):
            obj = os.path.join(OBJ, f"{tu}_{'bf16' if bf else 'f32'}.o")
            if force or _stale(obj, [src] + hdrs):
                jobs.append((src, obj, [f"-DSRWM_TIO_BF16={bf}"] + extra_all, verbose))
    for name in ("api",):
        src = os.path.join(CSRC, name + ".cu")
        if not os.path.exists(src):
            continue
        obj = os.path.join(OBJ, name + ".o")
        if force or _stale(obj, [src] + hdrs):
            jobs.append((src, obj, list(extra_all), verbose))
    logs = []
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for obj, rc, out in ex.map(_compile, jobs):
                logs.append((obj, out))
                if rc != 0:
                    sys.stderr.write(out)
                    raise RuntimeError(f"nvcc failed for {obj}")
    objs = sorted(os.path.join(OBJ, f) for f in os.listdir(OBJ) if f.endswith(".o"))
    with open(stamp, "w") as fh:
        fh.write(cur + "\n")
    if jobs or not os.path.exists(LIB):
        cmd = [_nvcc()] + ARCH + ["-shared", "-o", LIB] + objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    if verbose:
        for obj, out in logs:
            print("==", obj)
            print(out)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register / spill report")
    ap.add_argument("--tuning", action="store_true", help="also compile the tuning alternatives of configs.h")
    ap.add_argument("--product", action="store_true", help="compile only the configurations the library picks")
    ap.add_argument("--debug", action="store_true",
                    help="build libsrwm_b200_debug.so: row checks that report through a status word")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose, tuning=True if a.tuning else (False if a.product else None),
                debug=a.debug))
