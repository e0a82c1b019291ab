"""Build recipe for the test oracle (test infrastructure, not part of the shipped library).

* ``liboracle_cnn.so``  -- oracle/cnn_oracle.c compiled twice (fp32 symbols ``*_f32`` and fp64
  symbols ``*_f64``) with gcc, OpenMP, ``-ffp-contract=off``.
* ``_ref/libref_cnn.so`` -- the reference's own ``layer.cu`` + ``layer.h``, compiled unmodified
  from the reference checkout where it lies, together with oracle/ref_harness.cu.  Built only
  where the checkout exists; the resulting file is git-ignored and used prebuilt elsewhere.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle_cnn.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libref_cnn.so")
# The reference checkout: $CNN_REFERENCE_DIR, else a directory "reference" beside the repository.
# Where neither exists the prebuilt files under _ref/ are used as they are.
REFERENCE_CHECKOUT = os.environ.get(
    "CNN_REFERENCE_DIR", os.path.normpath(os.path.join(HERE, "..", "..", "reference")))


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "cnn_oracle.c")
    if not force and _newer(ORACLE_SO, [src, __file__]):
        return ORACLE_SO
    common = ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-ffp-contract=off",
              "-fno-fast-math", "-std=c11", "-Wall", "-c", src]
    o32 = os.path.join(HERE, "cnn_oracle_f32.o")
    o64 = os.path.join(HERE, "cnn_oracle_f64.o")
    _run(common + ["-DREAL=float", "-DSUFFIX=_f32", "-o", o32])
    _run(common + ["-DREAL=double", "-DSUFFIX=_f64", "-DREAL_IS_DOUBLE", "-o", o64])
    _run(["gcc", "-shared", "-fopenmp", "-o", ORACLE_SO, o32, o64, "-lm"])
    return ORACLE_SO


def build_reference(force: bool = False) -> str | None:
    """Compile the unmodified reference kernels; returns the .so path, or None when neither the
    reference checkout nor a prebuilt library is available."""
    layer_cu = os.path.join(REFERENCE_CHECKOUT, "layer.cu")
    harness = os.path.join(HERE, "ref_harness.cu")
    if not os.path.exists(layer_cu):
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, [layer_cu, harness, __file__]):
        return REF_SO
    if shutil.which("nvcc") is None:
        return REF_SO if os.path.exists(REF_SO) else None
    os.makedirs(REF_DIR, exist_ok=True)
    # The reference's Makefile passes no -arch (so nvcc would embed old-architecture code that is
    # JIT-compiled at load); the target architecture is given here so the comparison is fair.
    _run(["nvcc", "-I" + REFERENCE_CHECKOUT, "-gencode", "arch=compute_100a,code=sm_100a",
          "-Wno-deprecated-gpu-targets", "-shared", "-Xcompiler", "-fPIC",
          "-o", REF_SO, harness, layer_cu])
    return REF_SO


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_reference(force="--force" in sys.argv))
