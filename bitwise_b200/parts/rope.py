"""Rotary position encoding: the table of angles, built on the host.

Base frequencies as the reference computes them, ``inv_freq[i] = 1.0f / powf(theta,
(float)(2i) / (float)hd)`` in 32-bit (src/model.cpp:220-225), the angle ``(float)pos *
inv_freq[i]`` and its ``cosf`` / ``sinf`` (src/kernels.cpp:276-279), all through the C
library so that a CPU implementation calling the same functions sees the same bits; the
kernels only read the table.  The ``llama3`` rescaling of the frequencies is not in the
reference (tools/convert.py:59-60 rejects rope_scaling): wavelengths shorter than
``orig / high_freq_factor`` stay, longer than ``orig / low_freq_factor`` are divided by
``factor``, the band between is blended linearly; evaluated in 64-bit from the 32-bit base
value and rounded once.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import numpy as np
import torch

from .base import PositionEncoding, register_position_encoding

_libm = ctypes.CDLL("libm.so.6")
_libm.powf.restype = ctypes.c_float
_libm.powf.argtypes = [ctypes.c_float, ctypes.c_float]
for _n in ("cosf", "sinf"):
    getattr(_libm, _n).restype = ctypes.c_float
    getattr(_libm, _n).argtypes = [ctypes.c_float]


def inverse_frequencies(head_dim: int, theta: float, scaling=None) -> np.ndarray:
    half = head_dim // 2
    theta32 = float(np.float32(theta))
    inv = np.empty(half, dtype=np.float32)
    for i in range(half):
        expo = np.float32(np.float32(2 * i) / np.float32(head_dim))
        inv[i] = np.float32(1.0) / np.float32(_libm.powf(theta32, float(expo)))
    if scaling is None:
        return inv
    lo_wave = scaling.original_max_position_embeddings / scaling.low_freq_factor
    hi_wave = scaling.original_max_position_embeddings / scaling.high_freq_factor
    out = np.empty(half, dtype=np.float32)
    for i in range(half):
        f = float(inv[i])
        wavelen = 2.0 * math.pi / f
        if wavelen < hi_wave:
            v = f
        elif wavelen > lo_wave:
            v = f / scaling.factor
        else:
            smooth = (scaling.original_max_position_embeddings / wavelen - scaling.low_freq_factor) / (
                scaling.high_freq_factor - scaling.low_freq_factor)
            v = (1.0 - smooth) * f / scaling.factor + smooth * f
        out[i] = np.float32(v)
    return out


class RotaryEncoding(PositionEncoding):
    """cos / sin tables [positions, head_dim / 2] in float32, grown on demand."""
    graph_safe = True  # kernels only: a step through this part can be captured


    def __init__(self, head_dim: int, theta: float, scaling=None, positions: int = 0):
        if head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head size, got {head_dim}")
        self.head_dim = head_dim
        self.inv_freq = inverse_frequencies(head_dim, theta, scaling)
        self._cos = np.empty((0, head_dim // 2), dtype=np.float32)
        self._sin = np.empty((0, head_dim // 2), dtype=np.float32)
        self._device_tables = {}
        self._retired = []
        if positions:
            self.reserve(positions)

    def reserve(self, positions: int) -> None:
        """Make the table cover positions 0 .. positions-1."""
        have = self._cos.shape[0]
        if positions <= have:
            return
        half = self.head_dim // 2
        cos = np.empty((positions, half), dtype=np.float32)
        sin = np.empty((positions, half), dtype=np.float32)
        cos[:have], sin[:have] = self._cos, self._sin
        cosf, sinf = _libm.cosf, _libm.sinf
        for p in range(have, positions):
            pf = np.float32(p)
            for i in range(half):
                a = float(pf * self.inv_freq[i])  # one 32-bit multiply
                cos[p, i] = cosf(a)
                sin[p, i] = sinf(a)
        self._cos, self._sin = cos, sin
        self._retired.append(self._device_tables)  # captured graphs may still read the old tables
        self._device_tables = {}

    def max_positions(self) -> Optional[int]:
        return self._cos.shape[0]

    def rotary_tables(self, device):
        key = str(device)
        if key not in self._device_tables:
            self._device_tables[key] = (torch.from_numpy(self._cos).to(device),
                                        torch.from_numpy(self._sin).to(device))
        return self._device_tables[key]


register_position_encoding("rotary", RotaryEncoding)
