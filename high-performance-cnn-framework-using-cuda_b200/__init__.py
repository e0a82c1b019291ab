"""Python host side of the B200 CNN hot path: a ctypes mirror of the reference's operator surface.

The reference's interface for this path is the C++ header ``layer.h``: ``class Layer(M, N, O)``
with ``setOutput / clear / bp_clear`` and the kernels ``fp_preact_c1 ... apply_grad`` that the
caller launches itself (main.cu:55-123).  This module exposes the same names with the same
argument meaning on top of the C ABI in ``include/cnn_b200.h`` (``libcnn_b200.so``), plus the fused
network (``Net``) that replaces the launch sequences of main.cu.

There is no CPU fallback: importing works anywhere (so the symbol table can be checked), but every
compute call needs the CUDA library and a GPU and raises ``CnnError`` otherwise.

The directory name contains hyphens, so the package is loaded by file path; see
``__graft_entry__.load_package`` (it registers the module as ``hpcnn_b200``).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import numpy as np

from . import checkpoint, synth  # noqa: F401  (re-exported)

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# CNN_B200_LIBRARY names an instrumented build of the same library (build.py --define ... --out ...).
LIB_PATH = os.environ.get("CNN_B200_LIBRARY") or os.path.join(PKG_DIR, "libcnn_b200.so")
HEADER_PATH = os.path.join(PKG_DIR, "..", "include", "cnn_b200.h")

N_PARAMS = 2343
N_PARAMS_PADDED = 2368
IMAGE_ELEMS = 784
N_OUT = 10

# Parameter arena: name -> (offset, shape), in the reference's Layer::weight / Layer::bias layout.
PARAM_LAYOUT = {
    "c1.weight": (0, (6, 5, 5)),
    "c1.bias": (150, (6,)),
    "s1.weight": (156, (1, 4, 4)),
    "s1.bias": (172, (1,)),
    "f.weight": (173, (10, 6, 6, 6)),
    "f.bias": (2333, (10,)),
}


class CnnError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__("cnn_b200 error %d: %s" % (code, message))
        self.code = code


class LayerView(C.Structure):
    _fields_ = [("M", C.c_int), ("N", C.c_int), ("O", C.c_int),
                ("output", C.c_void_p), ("preact", C.c_void_p), ("bias", C.c_void_p),
                ("weight", C.c_void_p), ("d_output", C.c_void_p), ("d_preact", C.c_void_p),
                ("d_weight", C.c_void_p)]


_lib: Optional[C.CDLL] = None

_P = C.c_void_p
_PROTOTYPES = {
    "cnn_last_error": (C.c_char_p, []),
    "cnn_build_info": (C.c_char_p, []),
    "cnn_layer_create": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(_P)]),
    "cnn_layer_destroy": (C.c_int, [_P]),
    "cnn_layer_set_output": (C.c_int, [_P, _P]),
    "cnn_layer_clear": (C.c_int, [_P]),
    "cnn_layer_bp_clear": (C.c_int, [_P]),
    "cnn_layer_view_get": (C.c_int, [_P, C.POINTER(LayerView)]),
    "cnn_apply_step_function": (C.c_int, [_P, _P, C.c_int, _P]),
    "cnn_make_error": (C.c_int, [_P, _P, C.c_uint, C.c_int, _P]),
    "cnn_apply_grad": (C.c_int, [_P, _P, C.c_int, _P]),
    "cnn_fp_preact_c1": (C.c_int, [_P, _P, _P, _P]),
    "cnn_fp_bias_c1": (C.c_int, [_P, _P, _P]),
    "cnn_fp_preact_s1": (C.c_int, [_P, _P, _P, _P]),
    "cnn_fp_bias_s1": (C.c_int, [_P, _P, _P]),
    "cnn_fp_preact_f": (C.c_int, [_P, _P, _P, _P]),
    "cnn_fp_bias_f": (C.c_int, [_P, _P, _P]),
    "cnn_bp_weight_f": (C.c_int, [_P, _P, _P, _P]),
    "cnn_bp_bias_f": (C.c_int, [_P, _P, _P]),
    "cnn_bp_output_s1": (C.c_int, [_P, _P, _P, _P]),
    "cnn_bp_preact_s1": (C.c_int, [_P, _P, _P, _P]),
    "cnn_bp_weight_s1": (C.c_int, [_P, _P, _P, _P]),
    "cnn_bp_bias_s1": (C.c_int, [_P, _P, _P]),
    "cnn_bp_output_c1": (C.c_int, [_P, _P, _P, _P]),
    "cnn_bp_preact_c1": (C.c_int, [_P, _P, _P, _P]),
    "cnn_bp_weight_c1": (C.c_int, [_P, _P, _P, _P]),
    "cnn_bp_bias_c1": (C.c_int, [_P, _P, _P]),
    "cnn_net_create": (C.c_int, [C.c_uint, C.POINTER(_P)]),
    "cnn_net_destroy": (C.c_int, [_P]),
    "cnn_net_set_params": (C.c_int, [_P, _P]),
    "cnn_net_get_params": (C.c_int, [_P, _P]),
    "cnn_net_params_device": (C.c_int, [_P, C.POINTER(_P)]),
    "cnn_net_set_fast_sigmoid": (C.c_int, [_P, C.c_int]),
    "cnn_net_set_option": (C.c_int, [_P, C.c_char_p, C.c_int]),
    "cnn_net_status": (C.c_int, [_P, C.POINTER(C.c_int)]),
    "cnn_forward_batched": (C.c_int, [_P, _P, C.c_long, _P, _P, _P]),
    "cnn_forward_batched_host": (C.c_int, [_P, _P, C.c_long, _P, _P]),
    "cnn_forward_batched_u8": (C.c_int, [_P, _P, C.c_long, _P, _P, _P]),
    "cnn_forward_batched_u8_host": (C.c_int, [_P, _P, C.c_long, _P, _P]),
    "cnn_synth_images": (C.c_int, [C.c_ulonglong, C.c_long, C.c_long, _P, _P, _P]),
    "cnn_wide_param_count": (C.c_int, [C.c_int, C.c_int]),
    "cnn_wide_create": (C.c_int, [C.c_int, C.c_int, C.POINTER(_P)]),
    "cnn_wide_destroy": (C.c_int, [_P]),
    "cnn_wide_set_params": (C.c_int, [_P, _P]),
    "cnn_wide_get_params": (C.c_int, [_P, _P]),
    "cnn_wide_set_option": (C.c_int, [_P, C.c_char_p, C.c_int]),
    "cnn_wide_status": (C.c_int, [_P, C.POINTER(C.c_int)]),
    "cnn_wide_forward": (C.c_int, [_P, _P, C.c_long, _P, _P, _P]),
    "cnn_wide_grad_batch": (C.c_int, [_P, _P, _P, C.c_long, _P, _P]),
    "cnn_wide_apply_update": (C.c_int, [_P, _P, C.c_float, _P]),
    "cnn_copy_to_host": (C.c_int, [_P, _P, C.c_size_t]),
    "cnn_copy_to_device": (C.c_int, [_P, _P, C.c_size_t]),
    "cnn_grad_batch": (C.c_int, [_P, _P, _P, C.c_long, _P, _P]),
    "cnn_grad_batch_noalloc": (C.c_int, [_P, _P, _P, C.c_long, _P, _P]),
    "cnn_grad_batch_noalloc_status": (C.c_int, [_P]),
    "cnn_dp_create": (C.c_int, [_P, C.c_int, C.c_int, C.POINTER(_P)]),
    "cnn_dp_destroy": (C.c_int, [_P]),
    "cnn_dp_export_handle": (C.c_int, [_P, _P]),
    "cnn_dp_connect": (C.c_int, [_P, _P]),
    "cnn_dp_local_buffer": (C.c_int, [_P, C.POINTER(_P)]),
    "cnn_dp_connect_pointers": (C.c_int, [_P, C.POINTER(_P)]),
    "cnn_dp_set_option": (C.c_int, [_P, C.c_char_p, C.c_int]),
    "cnn_dp_step": (C.c_int, [_P, _P, _P, C.c_long, C.c_float, _P, _P, C.c_float, _P]),
    "cnn_train_minibatch_dp": (C.c_int, [_P, _P, _P, C.c_long, C.c_long, C.c_int, C.c_float, _P, _P]),
    "cnn_net_save": (C.c_int, [_P, C.c_char_p]),
    "cnn_net_load": (C.c_int, [_P, C.c_char_p]),
    "cnn_wide_save": (C.c_int, [_P, C.c_char_p]),
    "cnn_wide_load": (C.c_int, [_P, C.c_char_p]),
    "cnn_apply_update": (C.c_int, [_P, _P, C.c_float, _P]),
    "cnn_train_minibatch": (C.c_int, [_P, _P, _P, C.c_long, C.c_int, C.c_int, C.c_float, _P, _P]),
    "cnn_train_sgd_persample": (C.c_int, [_P, _P, _P, C.c_long, C.c_int, C.c_float, C.c_float, _P, C.POINTER(C.c_int), _P]),
}


def exported_symbols() -> list:
    """Names of every entry point the Python side binds (checked against include/cnn_b200.h)."""
    return sorted(_PROTOTYPES)


def load_library() -> C.CDLL:
    """dlopen libcnn_b200.so (built in-tree by build.py) and bind every prototype.  Raises if the
    library is missing: there is deliberately nothing to fall back to."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise CnnError(-2, "libcnn_b200.so is not built (run build.py / __graft_entry__.build()); "
                           "there is no CPU fallback")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in _PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def _check(rc: int) -> None:
    if rc != 0:
        raise CnnError(rc, load_library().cnn_last_error().decode("utf-8", "replace"))


def _ptr(x) -> Optional[int]:
    """Device/host address of a torch tensor, numpy array, int or None."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return int(x.data_ptr())
    if isinstance(x, np.ndarray):
        return int(x.ctypes.data)
    if isinstance(x, C.c_void_p):
        return x.value
    raise TypeError("cannot take the address of %r" % type(x))


def _stream(stream) -> Optional[int]:
    if stream is None:
        return None
    if hasattr(stream, "cuda_stream"):
        return int(stream.cuda_stream)
    return int(stream)


def copy_to_host(dev_ptr: int, count: int, dtype=np.float32) -> np.ndarray:
    out = np.empty(count, dtype=dtype)
    if count:
        _check(load_library().cnn_copy_to_host(_ptr(out), dev_ptr, out.nbytes))
    return out


def copy_to_device(dev_ptr: int, arr: np.ndarray) -> None:
    arr = np.ascontiguousarray(arr)
    if arr.size:
        _check(load_library().cnn_copy_to_device(dev_ptr, _ptr(arr), arr.nbytes))


# ---------------------------------------------------------------------------------------------
# class Layer -- mirror of layer.h:14-35
# ---------------------------------------------------------------------------------------------
class Layer:
    """``Layer(M, N, O)``: M = fan-in per unit, N = units, O = output elements.  Owns seven device
    buffers with the reference's member names (as integer device addresses)."""

    _BUFFERS = ("output", "preact", "bias", "weight", "d_output", "d_preact", "d_weight")

    def __init__(self, M: int, N: int, O: int):
        lib = load_library()
        h = _P()
        _check(lib.cnn_layer_create(M, N, O, C.byref(h)))
        self._h = h
        v = LayerView()
        _check(lib.cnn_layer_view_get(h, C.byref(v)))
        self.M, self.N, self.O = v.M, v.N, v.O
        for b in self._BUFFERS:
            setattr(self, b, getattr(v, b) or 0)

    def _count(self, name: str) -> int:
        return {"output": self.O, "preact": self.O, "d_output": self.O, "d_preact": self.O,
                "bias": self.N, "weight": self.M * self.N, "d_weight": self.M * self.N}[name]

    def setOutput(self, data) -> None:  # noqa: N802  (reference spelling)
        arr = np.ascontiguousarray(np.asarray(data, dtype=np.float32).reshape(-1))
        if arr.size != self.O:
            raise ValueError("setOutput expects %d floats" % self.O)
        _check(load_library().cnn_layer_set_output(self._h, _ptr(arr)))

    def clear(self) -> None:
        _check(load_library().cnn_layer_clear(self._h))

    def bp_clear(self) -> None:
        _check(load_library().cnn_layer_bp_clear(self._h))

    def read(self, name: str) -> np.ndarray:
        return copy_to_host(getattr(self, name), self._count(name))

    def write(self, name: str, arr) -> None:
        arr = np.ascontiguousarray(np.asarray(arr, dtype=np.float32).reshape(-1))
        if arr.size != self._count(name):
            raise ValueError("%s holds %d floats" % (name, self._count(name)))
        copy_to_device(getattr(self, name), arr)

    def close(self) -> None:
        if getattr(self, "_h", None) is not None:
            load_library().cnn_layer_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---------------------------------------------------------------------------------------------
# Per-operator entry points, reference names and argument order (layer.h:40-62)
# ---------------------------------------------------------------------------------------------
def _op(name, nptr):
    def call(*args, stream=None):
        if len(args) != nptr:
            raise TypeError("%s takes %d pointer arguments" % (name, nptr))
        fn = getattr(load_library(), "cnn_" + name)
        _check(fn(*[_ptr(a) for a in args], _stream(stream)))
    call.__name__ = name
    call.__doc__ = "Reference operator %s (layer.h) through the C ABI." % name
    return call


def apply_step_function(input, output, N, stream=None):  # noqa: A002
    _check(load_library().cnn_apply_step_function(_ptr(input), _ptr(output), int(N), _stream(stream)))


def makeError(err, output, Y, N, stream=None):  # noqa: N802
    _check(load_library().cnn_make_error(_ptr(err), _ptr(output), int(Y), int(N), _stream(stream)))


def apply_grad(output, grad, N, stream=None):
    _check(load_library().cnn_apply_grad(_ptr(output), _ptr(grad), int(N), _stream(stream)))


fp_preact_c1 = _op("fp_preact_c1", 3)
fp_bias_c1 = _op("fp_bias_c1", 2)
fp_preact_s1 = _op("fp_preact_s1", 3)
fp_bias_s1 = _op("fp_bias_s1", 2)
fp_preact_f = _op("fp_preact_f", 3)
fp_bias_f = _op("fp_bias_f", 2)
bp_weight_f = _op("bp_weight_f", 3)
bp_bias_f = _op("bp_bias_f", 2)
bp_output_s1 = _op("bp_output_s1", 3)
bp_preact_s1 = _op("bp_preact_s1", 3)
bp_weight_s1 = _op("bp_weight_s1", 3)
bp_bias_s1 = _op("bp_bias_s1", 2)
bp_output_c1 = _op("bp_output_c1", 3)
bp_preact_c1 = _op("bp_preact_c1", 3)
bp_weight_c1 = _op("bp_weight_c1", 3)
bp_bias_c1 = _op("bp_bias_c1", 2)


# ---------------------------------------------------------------------------------------------
# Fused network
# ---------------------------------------------------------------------------------------------
class Net:
    """The reference's four-layer net (main.cu:17-20) as one parameter arena with fused kernels.

    ``seed`` seeds the C library's rand() before the parameters are drawn in the reference's
    order, so ``Net(0)`` starts from the reference binary's own initial parameters."""

    def __init__(self, seed: int = 0):
        lib = load_library()
        h = _P()
        _check(lib.cnn_net_create(seed, C.byref(h)))
        self._h = h

    # -- parameters ---------------------------------------------------------------------------
    def set_params(self, params) -> None:
        arr = np.ascontiguousarray(np.asarray(params, dtype=np.float32).reshape(-1))
        if arr.size != N_PARAMS:
            raise ValueError("parameter arena holds %d floats" % N_PARAMS)
        _check(load_library().cnn_net_set_params(self._h, _ptr(arr)))

    def get_params(self) -> np.ndarray:
        out = np.empty(N_PARAMS, dtype=np.float32)
        _check(load_library().cnn_net_get_params(self._h, _ptr(out)))
        return out

    def params_device_ptr(self) -> int:
        p = _P()
        _check(load_library().cnn_net_params_device(self._h, C.byref(p)))
        return int(p.value)

    def set_fast_sigmoid(self, flavour) -> None:
        """Sigmoid flavour of the fused kernels: 0/False = the reference expression, anything else =
        reduced-argument ex2 + refined reciprocal (a few 1e-7 relative; the default)."""
        _check(load_library().cnn_net_set_fast_sigmoid(self._h, int(flavour)))

    def save(self, path: str) -> None:
        """Write the parameter arena as a checkpoint file (format: ``checkpoint.py``)."""
        _check(load_library().cnn_net_save(self._h, os.fsencode(path)))

    def load(self, path: str) -> None:
        """Read a checkpoint written by ``save`` (or ``checkpoint.write_checkpoint``) into the arena."""
        _check(load_library().cnn_net_load(self._h, os.fsencode(path)))

    def set_option(self, key: str, value: int) -> None:
        _check(load_library().cnn_net_set_option(self._h, key.encode(), int(value)))

    def status(self) -> int:
        s = C.c_int(0)
        _check(load_library().cnn_net_status(self._h, C.byref(s)))
        return s.value

    # -- inference ----------------------------------------------------------------------------
    def forward(self, d_images, n: int, d_out=None, d_argmax=None, stream=None) -> None:
        """Fused batched forward on device buffers: images [n,28,28] fp32 -> out [n,10] fp32,
        argmax [n] int32."""
        _check(load_library().cnn_forward_batched(self._h, _ptr(d_images), int(n), _ptr(d_out),
                                                  _ptr(d_argmax), _stream(stream)))

    def forward_host(self, h_images, n: int, h_out=None, h_argmax=None) -> None:
        """Same through host buffers (pinned memory gives asynchronous copies)."""
        _check(load_library().cnn_forward_batched_host(self._h, _ptr(h_images), int(n), _ptr(h_out),
                                                       _ptr(h_argmax)))

    def forward_u8(self, d_pixels, n: int, d_out=None, d_argmax=None, stream=None) -> None:
        """Fused forward on uint8 pixels [n,28,28] (IDX storage); same results as ``forward`` on
        ``pixels / 255.0``."""
        _check(load_library().cnn_forward_batched_u8(self._h, _ptr(d_pixels), int(n), _ptr(d_out),
                                                     _ptr(d_argmax), _stream(stream)))

    def forward_u8_host(self, h_pixels, n: int, h_out=None, h_argmax=None) -> None:
        _check(load_library().cnn_forward_batched_u8_host(self._h, _ptr(h_pixels), int(n), _ptr(h_out),
                                                          _ptr(h_argmax)))

    # -- training -----------------------------------------------------------------------------
    def grad_batch(self, d_images, d_labels, n: int, d_grad, stream=None) -> None:
        """Summed per-sample gradients of n images at the current parameters into d_grad
        (2368 floats: arena order, then zero padding; d_grad[2344] = sum of ||delta_f||_2)."""
        _check(load_library().cnn_grad_batch(self._h, _ptr(d_images), _ptr(d_labels), int(n),
                                             _ptr(d_grad), _stream(stream)))

    def apply_update(self, d_grad, scale: float, stream=None) -> None:
        """params += scale * d_grad[0:2343]."""
        _check(load_library().cnn_apply_update(self._h, _ptr(d_grad), float(scale), _stream(stream)))

    def train_minibatch(self, d_images, d_labels, n: int, batch: int, epochs: int, dt: float = 0.1,
                        d_mean_err=None, stream=None) -> None:
        _check(load_library().cnn_train_minibatch(self._h, _ptr(d_images), _ptr(d_labels), int(n),
                                                  int(batch), int(epochs), float(dt),
                                                  _ptr(d_mean_err), _stream(stream)))

    def train_sgd_persample(self, d_images, d_labels, n: int, epochs: int, dt: float = 0.1,
                            threshold: float = -1.0, stream=None):
        """learn() (main.cu:125-170) in one persistent kernel; returns (epochs_run, mean_err[])."""
        mean_err = np.zeros(max(epochs, 1), dtype=np.float32)
        ran = C.c_int(0)
        _check(load_library().cnn_train_sgd_persample(self._h, _ptr(d_images), _ptr(d_labels), int(n),
                                                      int(epochs), float(dt), float(threshold),
                                                      _ptr(mean_err), C.byref(ran), _stream(stream)))
        return ran.value, mean_err[:ran.value]

    def close(self) -> None:
        if getattr(self, "_h", None) is not None:
            load_library().cnn_net_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DataParallel:
    """Minibatch SGD of a ``Net`` across the GPUs of one box with the gradient exchange fused into
    the update kernel (``cnn_dp_*``): one instance per rank, each on its own device.

    ``exchange`` is a callable that takes this rank's 64-byte handle and returns the list of all
    ranks' handles in rank order (e.g. ``torch.distributed.all_gather_object``); it is not needed
    for a single rank."""

    HANDLE_BYTES = 64

    def __init__(self, net: "Net", rank: int = 0, world: int = 1, exchange=None):
        lib = load_library()
        self.net, self.rank, self.world = net, rank, world
        h = _P()
        _check(lib.cnn_dp_create(net._h, rank, world, C.byref(h)))
        self._h = h
        if world > 1:
            if exchange is None:
                raise ValueError("exchange is required when world > 1")
            mine = (C.c_ubyte * self.HANDLE_BYTES)()
            _check(lib.cnn_dp_export_handle(self._h, C.cast(mine, _P)))
            handles = exchange(bytes(mine))
            if len(handles) != world or any(len(x) != self.HANDLE_BYTES for x in handles):
                raise ValueError("exchange must return one %d-byte handle per rank" % self.HANDLE_BYTES)
            blob = (C.c_ubyte * (self.HANDLE_BYTES * world)).from_buffer_copy(b"".join(handles))
            _check(lib.cnn_dp_connect(self._h, C.cast(blob, _P)))
        else:
            _check(lib.cnn_dp_connect(self._h, None))

    def set_option(self, key: str, value: int) -> None:
        _check(load_library().cnn_dp_set_option(self._h, key.encode(), int(value)))

    def step(self, d_images, d_labels, n_local: int, scale: float, d_grad_sum=None, d_mean_err=None,
             err_scale: float = 0.0, stream=None) -> None:
        _check(load_library().cnn_dp_step(self._h, _ptr(d_images), _ptr(d_labels), int(n_local), float(scale),
                                          _ptr(d_grad_sum), _ptr(d_mean_err), float(err_scale), _stream(stream)))

    def train_minibatch(self, d_images, d_labels, n: int, global_batch: int, epochs: int, dt: float = 0.1,
                        d_mean_err=None, stream=None) -> None:
        """Every rank passes the same n images; see ``cnn_train_minibatch_dp``."""
        _check(load_library().cnn_train_minibatch_dp(self._h, _ptr(d_images), _ptr(d_labels), int(n),
                                                     int(global_batch), int(epochs), float(dt),
                                                     _ptr(d_mean_err), _stream(stream)))

    def close(self) -> None:
        if getattr(self, "_h", None) is not None:
            load_library().cnn_dp_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class WideNet:
    """The widened variant of the same topology (H x H input, F maps; benchmark configuration 5 is
    H = 56, F = 64).  Parameters start at zero; set them with ``set_params``."""

    def __init__(self, H: int = 56, F: int = 64):
        lib = load_library()
        self.H, self.F = H, F
        self.n_params = int(lib.cnn_wide_param_count(H, F))
        self.n_padded = ((self.n_params + 2 + 31) // 32) * 32
        h = _P()
        _check(lib.cnn_wide_create(H, F, C.byref(h)))
        self._h = h

    def set_params(self, params) -> None:
        arr = np.ascontiguousarray(np.asarray(params, dtype=np.float32).reshape(-1))
        if arr.size != self.n_params:
            raise ValueError("parameter arena holds %d floats" % self.n_params)
        _check(load_library().cnn_wide_set_params(self._h, _ptr(arr)))

    def get_params(self) -> np.ndarray:
        out = np.empty(self.n_params, dtype=np.float32)
        _check(load_library().cnn_wide_get_params(self._h, _ptr(out)))
        return out

    def set_option(self, key: str, value: int) -> None:
        _check(load_library().cnn_wide_set_option(self._h, key.encode(), int(value)))

    def save(self, path: str) -> None:
        _check(load_library().cnn_wide_save(self._h, os.fsencode(path)))

    def load(self, path: str) -> None:
        _check(load_library().cnn_wide_load(self._h, os.fsencode(path)))

    def status(self) -> int:
        s = C.c_int(0)
        _check(load_library().cnn_wide_status(self._h, C.byref(s)))
        return s.value

    def forward(self, d_images, n: int, d_out=None, d_argmax=None, stream=None) -> None:
        _check(load_library().cnn_wide_forward(self._h, _ptr(d_images), int(n), _ptr(d_out), _ptr(d_argmax),
                                               _stream(stream)))

    def grad_batch(self, d_images, d_labels, n: int, d_grad, stream=None) -> None:
        _check(load_library().cnn_wide_grad_batch(self._h, _ptr(d_images), _ptr(d_labels), int(n), _ptr(d_grad),
                                                  _stream(stream)))

    def apply_update(self, d_grad, scale: float, stream=None) -> None:
        _check(load_library().cnn_wide_apply_update(self._h, _ptr(d_grad), float(scale), _stream(stream)))

    def close(self) -> None:
        if getattr(self, "_h", None) is not None:
            load_library().cnn_wide_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def grad_batch_noalloc(d_params, d_images, d_labels, n: int, d_grad, stream=None) -> None:
    """Summed gradient of n images at the parameters in ``d_params`` (2343 device floats) into
    ``d_grad`` (2368 device floats), for callers that may not allocate device memory: no ``Net`` is
    involved and the call allocates nothing (its scratch is a fixed array inside the library).  At
    most 65,536 images per call; calls that can overlap on the GPU share that array and race."""
    _check(load_library().cnn_grad_batch_noalloc(_ptr(d_params), _ptr(d_images), _ptr(d_labels), int(n),
                                                 _ptr(d_grad), _stream(stream)))


def grad_batch_noalloc_status(stream=None) -> None:
    """Waits for ``stream`` and raises ``CnnError`` (code -3) if a ``grad_batch_noalloc`` call on the
    current device gave up a bounded wait since the last query.  Allocates nothing."""
    _check(load_library().cnn_grad_batch_noalloc_status(_stream(stream)))


PHASE_CLOCK_STAMPS = ("top of the loop", "convolution + 8 sigmoids", "at barrier A", "subsample + FC partials sent",
                      "exchange landed", "output layer", "deltas + gradient terms", "at barrier B2", "at barrier E")


def persample_phase_clocks():
    """Per-warp sums of the SM clock at each stamp of the per-sample cluster kernel's loop, as a
    float64 array [4 warps][16 stamps] (CTA 0; warps 0-2 compute, warp 3 service; see
    PHASE_CLOCK_STAMPS), accumulated over the samples of the last run.  Only a library built with
    ``build.py --define CNN_PHASE_CLOCKS`` exports it; returns None otherwise."""
    lib = load_library()
    try:
        fn = lib.cnn_debug_phase_clocks8
    except AttributeError:
        return None
    out = (C.c_longlong * 64)()
    fn.restype = C.c_int
    _check(fn(out))
    return np.array(out[:], dtype=np.float64).reshape(4, 16)


def forward_tc_phase_clocks():
    """The same for the tensor-core forward kernel: float64 [16 warps][16 stamps] of CTA 0 of the last
    launch (warp 0 finisher, 1 MMA issue, 2-3 loaders, 4-15 epilogue), or None without the
    instrumented build."""
    lib = load_library()
    try:
        fn = lib.cnn_debug_phase_clocks_tc
    except AttributeError:
        return None
    out = (C.c_longlong * 256)()
    fn.restype = C.c_int
    _check(fn(out))
    return np.array(out[:], dtype=np.float64).reshape(16, 16)


def synth_images_device(seed: int, first_index: int, n: int, d_images, d_labels=None, stream=None) -> None:
    """Fill device buffers with synthetic images (and labels) -- same values as synth.synth_images."""
    _check(load_library().cnn_synth_images(int(seed), int(first_index), int(n), _ptr(d_images),
                                           _ptr(d_labels), _stream(stream)))
