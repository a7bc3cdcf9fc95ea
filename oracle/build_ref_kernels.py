"""Build the reference's own CUDA extensions, unmodified, into oracle/_ref/ (TEST INFRASTRUCTURE).

    python oracle/build_ref_kernels.py --reference /path/to/modern-srwm

Compiles ``supervised_learning/self_ref_v0/self_ref_v0.cu`` and
``supervised_learning/fast_weight/fast_weight_cuda.cu`` where they lie (no source is copied)
with ``torch.utils.cpp_extension.load`` for sm_100a, the same way the reference's packages
do at import time (self_ref_v0/__init__.py:19-27, fast_weight/__init__.py:17-20), but with
the build directory set to ``oracle/_ref/<name>/``.  nvcc cross-compiles, so this runs on a
machine without a GPU; the resulting pybind modules are loaded on a GPU machine by
``oracle/ref_kernels.py``.  They serve two purposes only: a GPU-vs-GPU parity check
against the reference's real kernels inside their valid envelope (SRWM: d_head <= 27 and
L within one shared-memory time chunk; delta: any L), and a "reference kernels on the same
B200" timing.  Nothing shipped imports them.
"""
import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

JOBS = [
    ("ref_self_ref", "supervised_learning/self_ref_v0/self_ref_v0.cu", ["--ftemplate-depth=1024"]),
    ("ref_fast_weight", "supervised_learning/fast_weight/fast_weight_cuda.cu", []),
]


def built():
    return all(os.path.exists(os.path.join(OUT, name, name + ".so")) for name, _, _ in JOBS)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("MODERN_SRWM_REFERENCE", os.path.join(HERE, "..", "..", "reference")),
                    help="root of the upstream modern-srwm checkout")
    args = ap.parse_args()
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load
    for name, rel, flags in JOBS:
        src = os.path.join(args.reference, rel)
        bdir = os.path.join(OUT, name)
        os.makedirs(bdir, exist_ok=True)
        print("building", name, "from", src, flush=True)
        load(name=name, sources=[src], build_directory=bdir, extra_cuda_cflags=flags, verbose=False,
             is_python_module=False)
        print("  ->", [f for f in os.listdir(bdir) if f.endswith(".so")], flush=True)


if __name__ == "__main__":
    main()
