"""In-tree build of libcnn_b200.so (the C-ABI library) with nvcc for sm_100a.

Usage: ``python build.py [--force] [--verbose]`` or ``build_library()`` from Python.
nvcc cross-compiles without a GPU; the resulting shared object sits next to this file.

``python build.py --define NAME [--define NAME2 ...] --out PATH`` builds an instrumented copy of
the library (for example ``--define CNN_PHASE_CLOCKS``, which compiles the per-sample kernel's
clock stamps in) into PATH with its objects in a directory of their own; the package loads it when
the environment variable CNN_B200_LIBRARY names it.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libcnn_b200.so")
OBJ_DIR = os.path.join(PKG_DIR, "build")

SOURCES = ["layer_abi.cu", "net.cu", "checkpoint.cu", "fused_forward.cu", "forward_tc.cu", "fused_train.cu", "dp_exchange.cu",
           "persample_cluster8.cu", "wide.cu", "wide_tc.cu", "wide_grad_tc.cu", "synth.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--extended-lambda",
    "-Xcompiler", "-fPIC",
]


def _deps() -> list[str]:
    out = [os.path.abspath(__file__)]
    for root, _, files in os.walk(CSRC):
        out += [os.path.join(root, f) for f in files if f.endswith((".cu", ".cuh", ".h"))]
    out.append(os.path.join(PKG_DIR, "..", "include", "cnn_b200.h"))
    return out


def _up_to_date() -> bool:
    if not os.path.exists(LIB_PATH):
        return False
    t = os.path.getmtime(LIB_PATH)
    return all(os.path.getmtime(d) <= t for d in _deps() if os.path.exists(d))


def _compile(src: str, verbose: bool, obj_dir: str = OBJ_DIR, defines: tuple[str, ...] = ()) -> tuple[str, str]:
    obj = os.path.join(obj_dir, os.path.splitext(src)[0] + ".o")
    cmd = ["nvcc"] + NVCC_FLAGS + ["-D" + d for d in defines] + (["-Xptxas", "-v"] if verbose else []) + [
        "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    return obj, r.stderr


def build_library(force: bool = False, verbose: bool = False, defines: tuple[str, ...] = (),
                  out: str | None = None) -> str:
    """Compile every CUDA source of the package for sm_100a; returns the library path.

    With `defines` and `out` an instrumented copy is built into `out` (always from scratch)."""
    if defines or out:
        if not out:
            raise ValueError("an instrumented build needs its own output path (out=...)")
        return _build(verbose, tuple(defines), os.path.abspath(out), os.path.abspath(out) + ".objs")
    if not force and _up_to_date():
        return LIB_PATH
    if shutil.which("nvcc") is None:
        if os.path.exists(LIB_PATH):
            return LIB_PATH
        raise RuntimeError("nvcc not found and no prebuilt libcnn_b200.so present")
    return _build(verbose, (), LIB_PATH, OBJ_DIR)


def _build(verbose: bool, defines: tuple[str, ...], lib_path: str, obj_dir: str) -> str:
    os.makedirs(obj_dir, exist_ok=True)
    sources = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(sources)) as ex:
        results = list(ex.map(lambda s: _compile(s, verbose, obj_dir, defines), sources))
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", lib_path] + [o for o, _ in results]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    return lib_path


def _args_after(flag: str) -> list[str]:
    return [sys.argv[i + 1] for i, a in enumerate(sys.argv[:-1]) if a == flag]


if __name__ == "__main__":
    outs = _args_after("--out")
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
                        defines=tuple(_args_after("--define")), out=outs[-1] if outs else None))
