"""CPU tests of the boundary and the host logic: the C-ABI library loads and exports every symbol
the header declares, the Python mirror binds all of them, the synthetic generator is
deterministic, and the sharding arithmetic tiles its range."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "cnn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cnn_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_reference_operator_surface():
    syms = declared_symbols()
    for op in ["apply_step_function", "make_error", "apply_grad", "fp_preact_c1", "fp_bias_c1",
               "fp_preact_s1", "fp_bias_s1", "fp_preact_f", "fp_bias_f", "bp_weight_f", "bp_bias_f",
               "bp_output_s1", "bp_preact_s1", "bp_weight_s1", "bp_bias_s1", "bp_output_c1",
               "bp_preact_c1", "bp_weight_c1", "bp_bias_c1"]:
        assert "cnn_" + op in syms, op
    for fn in ["layer_create", "layer_destroy", "layer_set_output", "layer_clear", "layer_bp_clear"]:
        assert "cnn_" + fn in syms


def test_library_exports_every_declared_symbol(built):
    lib = ctypes.CDLL(built.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), "libcnn_b200.so does not export %s" % name


def test_python_mirror_binds_every_declared_symbol(built):
    assert sorted(built.exported_symbols()) == declared_symbols()
    built.load_library()
    assert b"sm_100a" in built.load_library().cnn_build_info()


def test_python_mirror_keeps_reference_names(pkg):
    for name in ["Layer", "apply_step_function", "makeError", "apply_grad", "fp_preact_c1",
                 "fp_bias_c1", "fp_preact_s1", "fp_bias_s1", "fp_preact_f", "fp_bias_f",
                 "bp_weight_f", "bp_bias_f", "bp_output_s1", "bp_preact_s1", "bp_weight_s1",
                 "bp_bias_s1", "bp_output_c1", "bp_preact_c1", "bp_weight_c1", "bp_bias_c1"]:
        assert hasattr(pkg, name), name
    for m in ["setOutput", "clear", "bp_clear"]:
        assert hasattr(pkg.Layer, m)


def test_invalid_arguments_are_rejected_without_a_gpu(built):
    lib = built.load_library()
    assert lib.cnn_forward_batched(None, None, 0, None, None, None) == -1
    assert b"NULL net" in lib.cnn_last_error()
    assert lib.cnn_apply_step_function(None, None, 4, None) == -1
    assert lib.cnn_layer_clear(None) == -1
    assert lib.cnn_net_set_option(None, b"x", 0) == -1


def test_no_cpu_fallback_in_the_product(pkg):
    """The package never imports the oracle."""
    pkg_dir = os.path.dirname(pkg.__file__)
    for root, _, files in os.walk(pkg_dir):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(root, f)).read()
                assert "oracle_binding" not in text and "liboracle" not in text, f


def test_synth_is_deterministic_and_mnist_shaped(pkg):
    a, la = pkg.synth.synth_images(1, 500)
    b, lb = pkg.synth.synth_images(1, 500)
    assert np.array_equal(a, b) and np.array_equal(la, lb)
    assert a.shape == (500, 28, 28) and a.dtype == np.float32 and la.dtype == np.uint32
    zero = float((a == 0).mean())
    assert 0.78 <= zero <= 0.82, zero
    nz = a[a > 0]
    assert nz.min() >= np.float32(128 / 255.0) and nz.max() <= 1.0
    assert la.min() >= 0 and la.max() <= 9
    # offsets index the same stream
    c, lc = pkg.synth.synth_images(1, 100, first_index=400)
    assert np.array_equal(c, a[400:]) and np.array_equal(lc, la[400:])
    # different sets differ
    d, _ = pkg.synth.synth_images(2, 10)
    assert not np.array_equal(d, a[:10])


def test_synth_params_range(pkg):
    p = pkg.synth.synth_params(0)
    assert p.shape == (2343,) and p.dtype == np.float32
    assert p.min() >= -0.5 and p.max() <= 0.5 and abs(float(p.mean())) < 0.02
    assert np.array_equal(p, pkg.synth.synth_params(0))
    assert not np.array_equal(p, pkg.synth.synth_params(1))


def test_u8_ingest_matches_reference_scaling(pkg):
    v = np.arange(256, dtype=np.uint8)
    f = pkg.synth.u8_to_float(v)
    assert np.array_equal(f, (v.astype(np.float64) / 255.0).astype(np.float32))


@pytest.mark.parametrize("n,world", [(0, 1), (1, 8), (7, 2), (65536, 8), (16777216, 8), (60000, 4), (10, 3)])
def test_shard_range_tiles(pkg, n, world):
    from hpcnn_b200 import parallel
    prev = 0
    sizes = []
    for r in range(world):
        lo, hi = parallel.shard_range(n, r, world)
        assert lo == prev and hi >= lo
        prev = hi
        sizes.append(hi - lo)
    assert prev == n and max(sizes) - min(sizes) <= 1


def test_batch_plan(pkg):
    from hpcnn_b200 import parallel
    plan = parallel.batch_plan(60000, 2048)
    assert plan[0] == (0, 2048) and plan[-1] == (59392, 608) and sum(s for _, s in plan) == 60000
    assert parallel.batch_plan(0, 4) == []
    with pytest.raises(ValueError):
        parallel.batch_plan(10, 0)
    with pytest.raises(ValueError):
        parallel.shard_range(10, 3, 3)


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 with nothing but the C library."""
    import subprocess
    src = tmp_path / "use_header.c"
    src.write_text('#include "cnn_b200.h"\nint main(void) { cnn_net* n = 0; (void)n; return CNN_OK; }\n')
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"),
                        "-fsyntax-only", str(src)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_instrumented_build_exports_the_phase_clock_readers(tmp_path):
    """`build.py --define CNN_PHASE_CLOCKS --out PATH` (the command the profile summaries give) builds a
    separate library that exports the clock-stamp readers of the three instrumented kernels; the in-tree
    library exports none of them."""
    import importlib.util
    import shutil
    if shutil.which("nvcc") is None:
        pytest.skip("nvcc not available")
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
    pkg_dir = [d for d in os.listdir(root) if d.endswith("_b200") and os.path.isdir(os.path.join(root, d))][0]
    spec = importlib.util.spec_from_file_location("b200_build", os.path.join(root, pkg_dir, "build.py"))
    build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(build)
    out = str(tmp_path / "libcnn_phase.so")
    assert build.build_library(defines=("CNN_PHASE_CLOCKS",), out=out) == out
    lib = ctypes.CDLL(out)
    plain = ctypes.CDLL(build.build_library())
    for name in ("cnn_debug_phase_clocks8", "cnn_debug_phase_clocks_tc", "cnn_debug_phase_clocks_wg"):
        assert hasattr(lib, name), name
        assert not hasattr(plain, name), name
