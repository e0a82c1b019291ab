"""ctypes bindings of the test oracle (oracle/liboracle_cnn.so) and of the unmodified reference
kernels (oracle/_ref/libref_cnn.so).  Test infrastructure: only tests, the smoke check and the
benchmark's CPU-baseline legs import this module."""
from __future__ import annotations

import ctypes as C
import importlib.util
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")

N_PARAMS = 2343
_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)


def _builder():
    spec = importlib.util.spec_from_file_location("hpcnn_b200_build_oracle",
                                                  os.path.join(ORACLE_DIR, "build_oracle.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


_oracle = None
_ref = None


class _Trace32(C.Structure):
    _names = ["c1_preact", "c1_output", "s1_preact", "s1_output", "f_preact", "f_output",
              "f_d_preact", "f_d_weight", "s1_d_output", "s1_d_preact", "s1_d_weight",
              "c1_d_output", "c1_d_preact", "c1_d_weight"]
    _fields_ = [(n, C.c_void_p) for n in _names]


def trace_sizes(H=28, F=6):
    Cc = H - 4
    P = Cc // 4
    S = F * P * P
    fcc = F * Cc * Cc
    return {"c1_preact": fcc, "c1_output": fcc, "s1_preact": S, "s1_output": S, "f_preact": 10,
            "f_output": 10, "f_d_preact": 10, "f_d_weight": 10 * S, "s1_d_output": S,
            "s1_d_preact": S, "s1_d_weight": 16, "c1_d_output": fcc, "c1_d_preact": fcc,
            "c1_d_weight": F * 25}


def oracle():
    global _oracle
    if _oracle is None:
        path = _builder().build_oracle()
        _oracle = C.CDLL(path)
    return _oracle


def param_count(H=28, F=6) -> int:
    return int(oracle().oracle_param_count_f32(H, F))


def _real(dtype):
    if dtype == np.float32:
        return "_f32", C.c_float
    if dtype == np.float64:
        return "_f64", C.c_double
    raise ValueError(dtype)


def _vp(a):
    return C.c_void_p(a.ctypes.data)


def forward_batch(params, images, H=28, F=6, threads=0, dtype=np.float32):
    """(out [n,10], argmax [n]) from the oracle."""
    suf, _ = _real(dtype)
    params = np.ascontiguousarray(params, dtype=dtype)
    images = np.ascontiguousarray(images, dtype=dtype).reshape(-1, H * H)
    n = images.shape[0]
    out = np.empty((n, 10), dtype=dtype)
    arg = np.empty((n,), dtype=np.int32)
    fn = getattr(oracle(), "oracle_forward_batch" + suf)
    fn.restype = None
    fn(C.c_int(H), C.c_int(F), _vp(params), _vp(images), C.c_long(n), _vp(out), _vp(arg), C.c_int(threads))
    return out, arg


def _make_trace(dtype, H, F):
    sizes = trace_sizes(H, F)
    arrays = {k: np.zeros(v, dtype=dtype) for k, v in sizes.items()}
    t = _Trace32()
    for k, a in arrays.items():
        setattr(t, k, a.ctypes.data)
    return t, arrays


def forward_trace(params, image, H=28, F=6, dtype=np.float32):
    """Every forward intermediate of one image, by the reference's Layer buffer names."""
    suf, _ = _real(dtype)
    params = np.ascontiguousarray(params, dtype=dtype)
    image = np.ascontiguousarray(image, dtype=dtype).reshape(-1)
    t, arrays = _make_trace(dtype, H, F)
    fn = getattr(oracle(), "oracle_forward" + suf)
    fn.restype = None
    fn(C.c_int(H), C.c_int(F), _vp(params), _vp(image), C.byref(t))
    return {k: arrays[k] for k in ("c1_preact", "c1_output", "s1_preact", "s1_output", "f_preact", "f_output")}


def sgd_step(params, image, label, dt=0.1, H=28, F=6, dtype=np.float32):
    """One reference SGD step: returns (new_params, err_norm, trace dict)."""
    suf, real = _real(dtype)
    p = np.array(params, dtype=dtype, copy=True)
    image = np.ascontiguousarray(image, dtype=dtype).reshape(-1)
    t, arrays = _make_trace(dtype, H, F)
    err = real(0)
    fn = getattr(oracle(), "oracle_sgd_step" + suf)
    fn.restype = None
    fn(C.c_int(H), C.c_int(F), _vp(p), _vp(image), C.c_uint(int(label)), real(dt), C.byref(err), C.byref(t))
    return p, float(err.value), arrays


def train_persample(params, images, labels, epochs, dt=0.1, threshold=-1.0, H=28, F=6, dtype=np.float32):
    """learn(): returns (params, mean_err[epochs_run], epochs_run)."""
    suf, real = _real(dtype)
    p = np.array(params, dtype=dtype, copy=True)
    images = np.ascontiguousarray(images, dtype=dtype).reshape(-1, H * H)
    labels = np.ascontiguousarray(labels, dtype=np.uint32)
    mean_err = np.zeros(max(epochs, 1), dtype=dtype)
    fn = getattr(oracle(), "oracle_train_persample" + suf)
    fn.restype = C.c_int
    ran = fn(C.c_int(H), C.c_int(F), _vp(p), _vp(images), _vp(labels), C.c_long(images.shape[0]),
             C.c_int(epochs), real(dt), real(threshold), _vp(mean_err))
    return p, mean_err[:ran], ran


def grad_batch(params, images, labels, H=28, F=6, threads=0, dtype=np.float32):
    """(G [n_params], err_sum): summed per-image gradients at fixed parameters."""
    suf, real = _real(dtype)
    params = np.ascontiguousarray(params, dtype=dtype)
    images = np.ascontiguousarray(images, dtype=dtype).reshape(-1, H * H)
    labels = np.ascontiguousarray(labels, dtype=np.uint32)
    G = np.zeros(param_count(H, F), dtype=dtype)
    err = real(0)
    fn = getattr(oracle(), "oracle_grad_batch" + suf)
    fn.restype = None
    fn(C.c_int(H), C.c_int(F), _vp(params), _vp(images), _vp(labels), C.c_long(images.shape[0]),
       _vp(G), C.byref(err), C.c_int(threads))
    return G, float(err.value)


def apply_update(params, G, dt, global_batch, dtype=np.float32):
    suf, real = _real(dtype)
    p = np.array(params, dtype=dtype, copy=True)
    G = np.ascontiguousarray(G, dtype=dtype)
    fn = getattr(oracle(), "oracle_apply_update" + suf)
    fn.restype = None
    fn(C.c_int(p.size), _vp(p), _vp(G), real(dt), real(global_batch))
    return p


def train_minibatch(params, images, labels, batch, epochs, dt=0.1, H=28, F=6, world=1, dtype=np.float32):
    """The library's minibatch rule on the oracle: batches in index order (the last may be
    smaller); with world > 1 each batch is split into `world` contiguous shards whose gradient
    vectors are added in rank order (what a sum-allreduce delivers)."""
    p = np.array(params, dtype=dtype, copy=True)
    images = np.ascontiguousarray(images, dtype=dtype).reshape(-1, H * H)
    n = images.shape[0]
    mean_err = []
    for _ in range(epochs):
        es = 0.0
        for first in range(0, n, batch):
            b = min(batch, n - first)
            G = None
            bounds = [first + (b * r) // world for r in range(world + 1)]
            for r in range(world):
                lo, hi = bounds[r], bounds[r + 1]
                if hi > lo:
                    g, e = grad_batch(p, images[lo:hi], labels[lo:hi], H, F, dtype=dtype)
                    es += e
                    G = g if G is None else (G + g).astype(dtype)
            p = apply_update(p, G, dt, b, dtype=dtype)
        mean_err.append(es / n)
    return p, np.array(mean_err, dtype=dtype)


# ------------------------------------------------------------------------------------------------
# The unmodified reference kernels (GPU only)
# ------------------------------------------------------------------------------------------------
REF_LAYERS = {"input": 0, "c1": 1, "s1": 2, "f": 3}
REF_BUFFERS = {"output": 0, "preact": 1, "bias": 2, "weight": 3, "d_output": 4, "d_preact": 5, "d_weight": 6}
REF_SIZES = {"input": (0, 0, 784), "c1": (25, 6, 3456), "s1": (16, 1, 216), "f": (216, 10, 10)}
REF_OPS = ["fp_preact_c1", "fp_bias_c1", "step_c1", "fp_preact_s1", "fp_bias_s1", "step_s1",
           "fp_preact_f", "fp_bias_f", "step_f", "makeError", "bp_weight_f", "bp_bias_f",
           "bp_output_s1", "bp_preact_s1", "bp_weight_s1", "bp_bias_s1", "bp_output_c1",
           "bp_preact_c1", "bp_weight_c1", "bp_bias_c1", "apply_grad_f", "apply_grad_s1",
           "apply_grad_c1"]


def reference_available() -> bool:
    return _builder().build_reference() is not None


class Reference:
    """The reference's own CUDA kernels (layer.cu, unmodified) behind oracle/ref_harness.cu."""

    def __init__(self, seed: int = 0):
        global _ref
        path = _builder().build_reference()
        if path is None:
            raise RuntimeError("oracle/_ref/libref_cnn.so is not available")
        if _ref is None:
            _ref = C.CDLL(path)
            _ref.ref_time_train.restype = C.c_double
            _ref.ref_time_classify.restype = C.c_double
            _ref.ref_read.restype = C.c_long
            _ref.ref_write.restype = C.c_long
        self.lib = _ref
        self.lib.ref_destroy()
        rc = self.lib.ref_create(C.c_uint(seed))
        if rc != 0:
            raise RuntimeError("ref_create failed: %d" % rc)

    def close(self):
        self.lib.ref_destroy()

    def _count(self, layer, buf):
        M, N, O = REF_SIZES[layer]
        return {"output": O, "preact": O, "d_output": O, "d_preact": O, "bias": N, "weight": M * N,
                "d_weight": M * N}[buf]

    def read(self, layer, buf):
        out = np.zeros(self._count(layer, buf), dtype=np.float32)
        n = self.lib.ref_read(REF_LAYERS[layer], REF_BUFFERS[buf], _vp(out))
        assert n == out.size, (layer, buf, n)
        return out

    def write(self, layer, buf, arr):
        arr = np.ascontiguousarray(arr, dtype=np.float32).reshape(-1)
        assert arr.size == self._count(layer, buf)
        self.lib.ref_write(REF_LAYERS[layer], REF_BUFFERS[buf], _vp(arr))

    def get_params(self):
        p = np.zeros(N_PARAMS, dtype=np.float32)
        self.lib.ref_get_params(_vp(p))
        return p

    def set_params(self, p):
        p = np.ascontiguousarray(p, dtype=np.float32)
        assert p.size == N_PARAMS
        self.lib.ref_set_params(_vp(p))

    def forward(self, image, grid=64, block=64):
        image = np.ascontiguousarray(image, dtype=np.float32).reshape(-1)
        rc = self.lib.ref_forward(_vp(image), grid, block)
        assert rc == 0, rc

    def train_step(self, image, label, grid=64, block=64):
        image = np.ascontiguousarray(image, dtype=np.float32).reshape(-1)
        err = C.c_float(0)
        rc = self.lib.ref_train_step(_vp(image), C.c_uint(int(label)), C.byref(err), grid, block)
        assert rc == 0, rc
        return float(err.value)

    def classify(self, image):
        image = np.ascontiguousarray(image, dtype=np.float32).reshape(-1)
        return int(self.lib.ref_classify(_vp(image)))

    def launch_op(self, name, grid=64, block=64, arg=0):
        rc = self.lib.ref_launch_op(REF_OPS.index(name), grid, block, C.c_uint(int(arg)))
        assert rc == 0, (name, rc)

    def time_train(self, images, labels):
        images = np.ascontiguousarray(images, dtype=np.float32).reshape(-1, 784)
        labels = np.ascontiguousarray(labels, dtype=np.uint32)
        me = C.c_float(0)
        sec = self.lib.ref_time_train(_vp(images), _vp(labels), C.c_long(images.shape[0]), C.byref(me))
        return float(sec), float(me.value)

    def time_classify(self, images):
        images = np.ascontiguousarray(images, dtype=np.float32).reshape(-1, 784)
        preds = np.zeros(images.shape[0], dtype=np.uint32)
        sec = self.lib.ref_time_classify(_vp(images), C.c_long(images.shape[0]), _vp(preds))
        return float(sec), preds
