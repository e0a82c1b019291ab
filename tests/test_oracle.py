"""CPU tests of the oracle: closed-form cases, an independent numpy restatement, fp32 vs fp64,
update semantics, edge cases, and the golden vectors recorded from the reference's CUDA kernels."""
import glob
import os

import numpy as np
import pytest

import numpy_model as nm
from conftest import rel_err, scaled_err

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_param_count(ob):
    assert ob.param_count(28, 6) == 2343
    assert ob.param_count(56, 64) == 64 * 25 + 64 + 16 + 1 + 10 * 64 * 13 * 13 + 10


def test_constant_network_closed_form(ob):
    # conv weights/bias 0 -> conv activation 0.5 everywhere; subsample weights 1, bias 0 ->
    # pre-activation 16*0.5 = 8; FC weights 0 and bias b -> output sigmoid(b).
    p = np.zeros(2343, dtype=np.float32)
    p[156:172] = 1.0
    p[2333:2343] = np.linspace(-2, 2, 10)
    x = np.random.default_rng(0).random((28, 28), dtype=np.float32)
    t = ob.forward_trace(p, x)
    assert np.all(t["c1_output"] == 0.5)
    assert np.allclose(t["s1_preact"], 8.0)
    assert np.allclose(t["s1_output"], 1 / (1 + np.exp(-8.0)), rtol=1e-6)
    assert np.allclose(t["f_output"], 1 / (1 + np.exp(-np.linspace(-2, 2, 10))), rtol=1e-6)


def test_conv_is_cross_correlation_without_flip(ob):
    # One lit pixel at (10, 12): preact[f][y][x] = W[f][10-y][12-x] inside the 5x5 support.
    rng = np.random.default_rng(1)
    p = np.zeros(2343, dtype=np.float32)
    W = rng.standard_normal((6, 5, 5)).astype(np.float32)
    p[0:150] = W.reshape(-1)
    x = np.zeros((28, 28), dtype=np.float32)
    x[10, 12] = 1.0
    z = ob.forward_trace(p, x)["c1_preact"].reshape(6, 24, 24)
    expect = np.zeros((6, 24, 24), dtype=np.float32)
    for y in range(24):
        for xx in range(24):
            i, j = 10 - y, 12 - xx
            if 0 <= i < 5 and 0 <= j < 5:
                expect[:, y, xx] = W[:, i, j]
    assert np.array_equal(z, expect)


def test_subsample_shares_one_filter_with_stride_four(ob):
    rng = np.random.default_rng(2)
    p = rng.uniform(-0.5, 0.5, 2343).astype(np.float32)
    x = rng.random((28, 28), dtype=np.float32)
    t = ob.forward_trace(p, x)
    ac = t["c1_output"].reshape(6, 24, 24).astype(np.float64)
    Ws = p[156:172].reshape(4, 4).astype(np.float64)
    zs = np.einsum("fpiqj,ij->fpq", ac.reshape(6, 6, 4, 6, 4), Ws) + float(p[172])
    assert scaled_err(t["s1_preact"].reshape(6, 6, 6), zs) < 2e-6


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_forward_matches_numpy_restatement(ob, pkg, seed):
    params = pkg.synth.synth_params(seed)
    images, _ = pkg.synth.synth_images(100 + seed, 8)
    for x in images:
        t = ob.forward_trace(params, x)
        a = nm.forward(params, x)
        assert scaled_err(t["c1_preact"], a["zc"].reshape(-1)) < 2e-6
        assert rel_err(t["c1_output"], a["ac"].reshape(-1)) < 1e-5
        assert rel_err(t["s1_output"], a["as_"].reshape(-1)) < 1e-5
        assert rel_err(t["f_output"], a["af"]) < 1e-5


def test_fp32_and_fp64_oracles_agree(ob, params0, data64):
    images, _ = data64
    o32, a32 = ob.forward_batch(params0, images)
    o64, a64 = ob.forward_batch(params0, images, dtype=np.float64)
    assert rel_err(o32, o64) < 1e-5
    top2 = np.sort(o64, axis=1)
    clear = (top2[:, -1] - top2[:, -2]) > 1e-5 * top2[:, -1]
    assert np.array_equal(a32[clear], a64[clear])


def test_gradient_matches_numpy_restatement(ob, params0, data64):
    images, labels = data64
    for x, y in zip(images[:6], labels[:6]):
        G, err = ob.grad_batch(params0, x[None], np.array([y]))
        Gn, errn, _ = nm.gradient(params0, x, int(y))
        assert scaled_err(G, Gn) < 1e-5
        for name, (off, shape) in {"Wc": (0, 150), "bc": (150, 6), "Ws": (156, 16), "bs": (172, 1),
                                   "Wf": (173, 2160), "bf": (2333, 10)}.items():
            assert scaled_err(G[off:off + shape], Gn[off:off + shape]) < 2e-5, name
        assert abs(err - errn) < 1e-5 * errn


def test_sgd_step_semantics(ob, params0, data64):
    """One step == params + dt * gradient (the update uses only pre-update parameters), and the
    output delta carries no sigmoid derivative."""
    images, labels = data64
    x, y = images[3], int(labels[3])
    p1, err, tr = ob.sgd_step(params0, x, y)
    G, err2 = ob.grad_batch(params0, x[None], np.array([y]))
    assert scaled_err(p1 - params0, 0.1 * G) < 1e-4
    assert abs(err - err2) < 1e-6
    onehot = np.zeros(10, dtype=np.float32)
    onehot[y] = 1
    assert np.array_equal(tr["f_d_preact"], onehot - tr["f_output"])
    assert np.allclose(tr["f_d_weight"].reshape(10, 216), np.outer(tr["f_d_preact"], tr["s1_output"]), rtol=1e-6)


def test_minibatch_of_one_is_the_per_sample_step(ob, params0, data64):
    images, labels = data64
    p_a, _, _ = ob.train_persample(params0, images[:5], labels[:5], 1)
    p_b, _ = ob.train_minibatch(params0, images[:5], labels[:5], batch=1, epochs=1)
    assert scaled_err(p_a, p_b) < 1e-5


def test_minibatch_world_split_is_rounding_equivalent(ob, params0, data64):
    images, labels = data64
    p1, e1 = ob.train_minibatch(params0, images, labels, batch=32, epochs=2, world=1)
    p2, e2 = ob.train_minibatch(params0, images, labels, batch=32, epochs=2, world=4)
    assert scaled_err(p1, p2) < 1e-5
    assert np.allclose(e1, e2, rtol=1e-5)


def test_training_reduces_error(ob, params0, pkg):
    images, labels = pkg.synth.synth_images(5, 300)
    _, mean_err, ran = ob.train_persample(params0, images, labels, 3)
    assert ran == 3 and mean_err[2] < mean_err[0]


def test_early_stop_threshold(ob, params0, data64):
    images, labels = data64
    _, mean_err, ran = ob.train_persample(params0, images[:10], labels[:10], 5, threshold=10.0)
    assert ran == 1 and len(mean_err) == 1


def test_argmax_lowest_index_wins_ties(ob):
    import ctypes as C
    lib = ob.oracle()
    v = np.array([0.1, 0.9, 0.9, 0.3, 0.9, 0, 0, 0, 0, 0], dtype=np.float32)
    assert lib.oracle_argmax10_f32(C.c_void_p(v.ctypes.data)) == 1
    v[:] = 0.5
    assert lib.oracle_argmax10_f32(C.c_void_p(v.ctypes.data)) == 0


def test_empty_batch(ob, params0):
    out, arg = ob.forward_batch(params0, np.zeros((0, 28, 28), dtype=np.float32))
    assert out.shape == (0, 10) and arg.shape == (0,)
    G, err = ob.grad_batch(params0, np.zeros((0, 28, 28), dtype=np.float32), np.zeros(0, dtype=np.uint32))
    assert np.all(G == 0) and err == 0


def test_widened_shape_runs_and_matches_numpy(ob):
    rng = np.random.default_rng(3)
    n = ob.param_count(56, 64)
    params = rng.uniform(-0.5, 0.5, n).astype(np.float32) * 0.2
    x = rng.random((56, 56)).astype(np.float32)
    out, _ = ob.forward_batch(params, x[None], H=56, F=64)
    a = nm.forward(params, x, H=56, F=64)
    assert rel_err(out[0], a["af"]) < 1e-4
    G, _ = ob.grad_batch(params, x[None], np.array([3]), H=56, F=64)
    Gn, _, _ = nm.gradient(params, x, 3, H=56, F=64)
    assert scaled_err(G, Gn) < 1e-4


# ---- golden vectors recorded from the reference's own CUDA kernels ------------------------------
def _golden_files():
    return sorted(glob.glob(os.path.join(GOLDEN, "reference_cuda_*.npz")))


@pytest.mark.skipif(not _golden_files(), reason="no golden vectors recorded yet")
@pytest.mark.parametrize("path", _golden_files())
def test_oracle_matches_reference_cuda_golden(ob, path):
    """The fixtures hold inputs and every Layer buffer produced by the unmodified reference kernels
    on a B200 (tests/golden/make_golden.py).  fp32 tolerance: the reference sums with atomics in a
    run-dependent order."""
    g = np.load(path)
    params, images, labels = g["params"], g["images"], g["labels"]
    for i in range(g["fwd_f_output"].shape[0]):
        t = ob.forward_trace(params, images[i])
        for name in ("c1_preact", "c1_output", "s1_preact", "s1_output", "f_preact", "f_output"):
            ref = g["fwd_" + name][i]
            if name.endswith("preact"):
                assert scaled_err(t[name], ref) < 2e-6, (i, name)
            else:
                assert rel_err(t[name], ref) < 1e-5, (i, name)
    # one SGD step from identical state
    for i in range(g["step_params_after"].shape[0]):
        p1, err, tr = ob.sgd_step(params, images[i], int(labels[i]))
        assert scaled_err(p1, g["step_params_after"][i]) < 1e-5, i
        assert scaled_err(p1 - params, g["step_params_after"][i] - params) < 1e-4, i
        assert abs(err - float(g["step_err"][i])) < 1e-5
        for name in ("f_d_preact", "f_d_weight", "s1_d_output", "s1_d_preact", "s1_d_weight",
                     "c1_d_output", "c1_d_preact", "c1_d_weight"):
            assert scaled_err(tr[name], g["step_" + name][i]) < 1e-5, (i, name)
    # a short trajectory
    if "traj_params" in g:
        n = int(g["traj_n"])
        p, mean_err, _ = ob.train_persample(params, images[:n], labels[:n], 1)
        assert scaled_err(p, g["traj_params"]) < 1e-4
        assert abs(float(mean_err[0]) - float(g["traj_mean_err"])) < 1e-5
    if "rand_init_params" in g:
        # glibc rand() sequence after srand(0): the reference binary's own initial parameters
        assert g["rand_init_params"].shape == (2343,)
