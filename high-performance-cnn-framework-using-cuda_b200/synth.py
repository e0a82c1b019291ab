"""Host (numpy) implementation of the synthetic data generator.

The reference trains and tests on the MNIST IDX files (main.cu:30-33), which cannot be had
offline; seeded synthetic images of the same shape (28x28), storage (uint8 pixel, consumed as
``pixel / 255.0`` like mnist.h:145) and label range (0..9) stand in.  This module mirrors, bit for
bit, the CUDA generator ``cnn_synth_images`` (csrc/synth.cu); see that file for the recipe.
"""
from __future__ import annotations

import numpy as np

_G = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
_DX = np.array([8, 7, 6, 3, 0, -3, -6, -7, -8, -7, -6, -3, 0, 3, 6, 7], dtype=np.int64)
_DY = np.array([0, 3, 6, 7, 8, 7, 6, 3, 0, -3, -6, -7, -8, -7, -6, -3], dtype=np.int64)

N_PARAMS = 2343
SIDE = 28


def mix64(z: np.ndarray) -> np.ndarray:
    """splitmix64 finaliser on uint64 arrays (wrap-around arithmetic)."""
    z = np.asarray(z, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        z = z ^ (z >> np.uint64(31))
    return z


def _base(seed: int, first_index: int, n: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        seed_mix = mix64(np.uint64(seed) + _G)
        idx = np.arange(first_index, first_index + n, dtype=np.uint64)
        return mix64(seed_mix + idx)


def synth_labels(seed: int, n: int, first_index: int = 0) -> np.ndarray:
    """Labels (uint32, 0..9) of images first_index .. first_index+n-1 of set ``seed``."""
    return (mix64(_base(seed, first_index, n)) % np.uint64(10)).astype(np.uint32)


def synth_pixels_u8(seed: int, n: int, first_index: int = 0) -> np.ndarray:
    """uint8 pixels [n, 28, 28]: zero canvas with 5..7 two-pixel-wide strokes of value 128..255."""
    base = _base(seed, first_index, n)
    cover = np.zeros((n, SIDE, SIDE), dtype=bool)
    rows = np.arange(n)
    with np.errstate(over="ignore"):
        n_strokes = 5 + (mix64(base + np.uint64(1)) % np.uint64(3)).astype(np.int64)
        for s in range(7):
            r = mix64(base + np.uint64(2 + s))
            x0 = 4 + ((r & np.uint64(0xFF)) % np.uint64(20)).astype(np.int64)
            y0 = 4 + (((r >> np.uint64(8)) & np.uint64(0xFF)) % np.uint64(20)).astype(np.int64)
            length = 10 + (((r >> np.uint64(16)) & np.uint64(0xFF)) % np.uint64(13)).astype(np.int64)
            d1 = ((r >> np.uint64(24)) & np.uint64(15)).astype(np.int64)
            bend = ((r >> np.uint64(28)) & np.uint64(1)).astype(np.int64)
            turn = (((r >> np.uint64(32)) & np.uint64(0xFF)) % np.uint64(5)).astype(np.int64)
            d2 = np.where(bend == 1, (d1 + turn + 14) & 15, d1)
            half = length // 2
            active_stroke = s < n_strokes
            for t in range(22):
                active = active_stroke & (t < length)
                if not active.any():
                    continue
                t1 = np.minimum(t, half)
                t2 = np.where(t < half, 0, t - half)
                X = x0 * 8 + t1 * _DX[d1] + t2 * _DX[d2]
                Y = y0 * 8 + t1 * _DY[d1] + t2 * _DY[d2]
                px, py = X >> 3, Y >> 3
                for b in (0, 1):
                    for a in (0, 1):
                        xx, yy = px + a, py + b
                        ok = active & (xx >= 0) & (xx < SIDE) & (yy >= 0) & (yy < SIDE)
                        cover[rows[ok], yy[ok], xx[ok]] = True
        pix = np.arange(SIDE * SIDE, dtype=np.uint64)[None, :]
        val = (np.uint64(128) + (mix64(base[:, None] + np.uint64(64) + pix) & np.uint64(127))).astype(np.uint8)
    out = np.where(cover.reshape(n, -1), val, np.uint8(0)).reshape(n, SIDE, SIDE)
    return out


def u8_to_float(pixels_u8: np.ndarray) -> np.ndarray:
    """The reference's ingest: pixel / 255.0 in double (mnist.h:145), then narrowed to float
    (main.cu:57-65)."""
    lut = (np.arange(256, dtype=np.float64) / 255.0).astype(np.float32)
    return lut[pixels_u8]


def synth_images(seed: int, n: int, first_index: int = 0):
    """(images float32 [n,28,28], labels uint32 [n]) of synthetic set ``seed``."""
    return u8_to_float(synth_pixels_u8(seed, n, first_index)), synth_labels(seed, n, first_index)


def synth_params(seed: int = 0, n_params: int = N_PARAMS) -> np.ndarray:
    """Parameter arena with every entry uniform in [-0.5, 0.5): 0.5 - u/2^24, u = top 24 bits of
    mix(mix(seed + G) + i)."""
    with np.errstate(over="ignore"):
        seed_mix = mix64(np.uint64(seed) + np.uint64(0xD1B54A32D192ED03))
        u = mix64(seed_mix + np.arange(n_params, dtype=np.uint64)) >> np.uint64(40)
    return (np.float32(0.5) - u.astype(np.float32) / np.float32(1 << 24)).astype(np.float32)
