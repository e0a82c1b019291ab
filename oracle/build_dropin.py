"""Builds the reference's own program twice (test infrastructure; needs the reference checkout):

* ``_ref/CNN_reference.exe``  main.cu + the reference's layer.cu           (the reference, unmodified)
* ``_ref/CNN_dropin.exe``     main.cu + this repository's compat/layer.cu  (the source-level drop-in)

main.cu and mnist.h are compiled from a scratch copy outside the repository, because
``#include "layer.h"`` resolves beside the including file first; nothing of the reference is copied
into the repository.  Where the checkout is absent the prebuilt files are used as they are."""
from __future__ import annotations

import os
import shutil
import subprocess
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF_DIR = os.path.join(HERE, "_ref")
# The reference checkout: $CNN_REFERENCE_DIR, else a directory "reference" beside the repository.
# Where neither exists the prebuilt files under _ref/ are used as they are.
REFERENCE_CHECKOUT = os.environ.get(
    "CNN_REFERENCE_DIR", os.path.normpath(os.path.join(HERE, "..", "..", "reference")))
COMPAT = os.path.join(ROOT, "high-performance-cnn-framework-using-cuda_b200", "compat")
TARGETS = {"reference": os.path.join(REF_DIR, "CNN_reference.exe"), "dropin": os.path.join(REF_DIR, "CNN_dropin.exe")}


def _run(cmd, cwd):
    r = subprocess.run(cmd, cwd=cwd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout[-2000:], r.stderr[-4000:]))


def build_dropin(force: bool = False):
    """Returns {"reference": path, "dropin": path}, or None when neither sources nor prebuilt files exist."""
    have = all(os.path.exists(p) for p in TARGETS.values())
    main_cu = os.path.join(REFERENCE_CHECKOUT, "main.cu")
    if not os.path.exists(main_cu) or shutil.which("nvcc") is None:
        return dict(TARGETS) if have else None
    deps = [main_cu, os.path.join(REFERENCE_CHECKOUT, "layer.cu"), os.path.join(COMPAT, "layer.cu"),
            os.path.join(COMPAT, "layer.h"), os.path.join(COMPAT, "..", "csrc", "layer_ops.cuh"), __file__]
    if have and not force:
        newest = max(os.path.getmtime(d) for d in deps)
        if all(os.path.getmtime(p) >= newest for p in TARGETS.values()):
            return dict(TARGETS)
    os.makedirs(REF_DIR, exist_ok=True)
    common = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-Wno-deprecated-gpu-targets",
              "-lcuda", "-lcudart", "-lcublas"]
    with tempfile.TemporaryDirectory() as tmp:
        # the reference as it is: all four sources side by side, its own Makefile line plus the arch
        ref_build = os.path.join(tmp, "ref")
        os.makedirs(ref_build)
        for f in ("main.cu", "mnist.h", "layer.cu", "layer.h"):
            shutil.copy(os.path.join(REFERENCE_CHECKOUT, f), ref_build)
        _run(common + ["-I.", "main.cu", "layer.cu", "-o", TARGETS["reference"]], ref_build)
        # the drop-in: the reference's main.cu and loader, this repository's operator layer
        drop_build = os.path.join(tmp, "drop")
        os.makedirs(drop_build)
        for f in ("main.cu", "mnist.h"):
            shutil.copy(os.path.join(REFERENCE_CHECKOUT, f), drop_build)
        _run(common + ["-std=c++17", "--extended-lambda", "--expt-relaxed-constexpr", "-I" + COMPAT,
                       "main.cu", os.path.join(COMPAT, "layer.cu"), "-o", TARGETS["dropin"]], drop_build)
    return dict(TARGETS)


if __name__ == "__main__":
    print(build_dropin(force=True))
