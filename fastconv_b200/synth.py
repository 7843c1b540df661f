"""Seeded synthetic tensors with the value distributions the benchmark configurations name.

Inputs are uniform in [-1, 1), weights He-normal N(0, sqrt(2 / (kh*kw*ic))), bias zero.  They stand
in for VGG-16 / ResNet-50 activations and weights (no dataset or checkpoint is used).  The
generator is a counter-based splitmix64 so the arrays do not depend on any library's RNG stream.
"""
from __future__ import annotations

import numpy as np

_U64 = np.uint64


def _splitmix64(idx: np.ndarray, seed: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = idx.astype(_U64) * _U64(0x9E3779B97F4A7C15) + _U64(seed & 0xFFFFFFFFFFFFFFFF) * _U64(0xD1B54A32D192ED03)
        z = z + _U64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> _U64(30))) * _U64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> _U64(27))) * _U64(0x94D049BB133111EB)
        return z ^ (z >> _U64(31))


def _unit(idx: np.ndarray, seed: int) -> np.ndarray:
    """float64 uniform in [0, 1) with 53 random bits"""
    return (_splitmix64(idx, seed) >> _U64(11)).astype(np.float64) * (1.0 / (1 << 53))


_CHUNK = 1 << 16  # elements per pass: the temporaries of a pass stay in cache, which is what makes large tensors cheap


def uniform(shape, seed: int, lo: float = -1.0, hi: float = 1.0) -> np.ndarray:
    n = int(np.prod(shape))
    out = np.empty(n, np.float32)
    for a in range(0, n, _CHUNK):
        b = min(n, a + _CHUNK)
        u = _unit(np.arange(a, b, dtype=_U64), seed)
        out[a:b] = (lo + (hi - lo) * u).astype(np.float32)
    return out.reshape(shape)


def normal(shape, seed: int, std: float = 1.0) -> np.ndarray:
    """Box-Muller on two independent counter streams."""
    n = int(np.prod(shape))
    out = np.empty(n, np.float32)
    for a in range(0, n, _CHUNK):
        b = min(n, a + _CHUNK)
        idx = np.arange(a, b, dtype=_U64)
        u1 = 1.0 - _unit(idx * _U64(2), seed)  # (0, 1]
        u2 = _unit(idx * _U64(2) + _U64(1), seed)
        z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
        out[a:b] = (z * std).astype(np.float32)
    return out.reshape(shape)


def conv_input(batch: int, ic: int, ih: int, iw: int, seed: int) -> np.ndarray:
    return uniform((batch, ic, ih, iw), seed)


def conv_weights(oc: int, ic: int, kh: int, kw: int, seed: int) -> np.ndarray:
    return normal((oc, ic, kh, kw), seed, std=float(np.sqrt(2.0 / (kh * kw * ic))))
