"""Parameter checkpoint files, host side (pure Python; the C ABI's ``cnn_net_save`` / ``cnn_net_load``
and ``cnn_wide_save`` / ``cnn_wide_load`` write and read the same bytes).

The reference keeps its parameters only in the device buffers of its four static ``Layer`` objects
(main.cu:17-20, filled at layer.cu:19-27) and loses them at exit.  A checkpoint is: a 32-byte
little-endian header -- magic ``CNNB200P``, version, kind (0 = the 28x28 net, 1 = widened), H, F,
parameter count, seed -- the arena as fp32 in the C ABI's order, and a 64-bit FNV-1a checksum of all
bytes before it.
"""
from __future__ import annotations

import struct

import numpy as np

MAGIC = b"CNNB200P"
VERSION = 1
_HEADER = struct.Struct("<8s6I")


class CheckpointError(ValueError):
    pass


def fnv1a(data: bytes) -> int:
    h = 1469598103934665603
    for b in data:
        h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def param_count(H: int = 28, F: int = 6) -> int:
    P = (H - 4) // 4
    return F * 25 + F + 16 + 1 + 10 * F * P * P + 10


def write_checkpoint(path: str, params, kind: int = 0, H: int = 28, F: int = 6, seed: int = 0) -> None:
    arr = np.ascontiguousarray(np.asarray(params, dtype="<f4").reshape(-1))
    if arr.size != param_count(H, F):
        raise CheckpointError("a net with H=%d, F=%d has %d parameters, got %d" % (H, F, param_count(H, F), arr.size))
    body = _HEADER.pack(MAGIC, VERSION, kind, H, F, arr.size, seed) + arr.tobytes()
    with open(path, "wb") as f:
        f.write(body + struct.pack("<Q", fnv1a(body)))


def read_checkpoint(path: str) -> dict:
    """Returns {"params": float32 array, "kind", "H", "F", "seed"}; raises CheckpointError on a bad
    magic, version, length or checksum."""
    with open(path, "rb") as f:
        data = f.read()
    if len(data) < _HEADER.size + 8:
        raise CheckpointError("file is shorter than a header")
    magic, version, kind, H, F, count, seed = _HEADER.unpack_from(data)
    if magic != MAGIC:
        raise CheckpointError("bad magic %r" % magic)
    if version != VERSION:
        raise CheckpointError("version %d, this reader handles %d" % (version, VERSION))
    want = _HEADER.size + 4 * count + 8
    if len(data) != want or count != param_count(H, F):
        raise CheckpointError("length %d does not fit %d parameters of H=%d, F=%d" % (len(data), count, H, F))
    (stored,) = struct.unpack_from("<Q", data, want - 8)
    if stored != fnv1a(data[:want - 8]):
        raise CheckpointError("checksum mismatch")
    params = np.frombuffer(data, dtype="<f4", count=count, offset=_HEADER.size).astype(np.float32)
    return {"params": params, "kind": kind, "H": H, "F": F, "seed": seed}
