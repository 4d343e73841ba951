"""Seeded random weights, and a model folder written from a configuration and a seed.

The reference's ``Model::random`` draws every tensor from one splitmix64 stream in a
fixed order (src/model.cpp:62-67,176-218).  Here the generator is counter based: the
value of element ``i`` of tensor ``name`` is a pure function of (seed, name, i), so a
tensor can be produced alone, in pieces, or in any order, and the plain test
implementation and the engine see the same bits because both read the written
folder.  Matrices are N(0, std) by Box-Muller in float64, then rounded once to the
storage dtype; norm weights are 1, or 1 + U(-jitter, jitter).  The 64-bit mixer is
the splitmix64 finaliser the reference also uses (src/engine.cpp:12-16).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable

import numpy as np
import torch

from .loader import INT_TABLE, KEEP32, ParamSpec
from .safetensors_io import write_safetensors

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _mix64(z: np.ndarray) -> np.ndarray:
    z = z.astype(np.uint64, copy=True)
    z ^= z >> np.uint64(30)
    z *= np.uint64(0xBF58476D1CE4E5B9)
    z ^= z >> np.uint64(27)
    z *= np.uint64(0x94D049BB133111EB)
    z ^= z >> np.uint64(31)
    return z


def _fnv1a64(data: bytes) -> int:
    h = 1469598103934665603
    for b in data:
        h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def tensor_key(seed: int, name: str) -> np.uint64:
    with np.errstate(over="ignore"):
        a = _mix64(np.array([(seed ^ 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF], dtype=np.uint64))
        b = _mix64(np.array([_fnv1a64(name.encode("utf-8"))], dtype=np.uint64))
    return np.uint64(a[0] ^ b[0])


def _uniform_pairs(key: np.uint64, start: int, count: int):
    with np.errstate(over="ignore"):
        idx = np.arange(start, start + count, dtype=np.uint64)
        a = _mix64(key ^ _mix64(idx * np.uint64(2)))
        b = _mix64(key ^ _mix64(idx * np.uint64(2) + np.uint64(1)))
    u1 = ((a >> np.uint64(11)).astype(np.float64) + 1.0) * 2.0 ** -53  # (0, 1]
    u2 = (b >> np.uint64(11)).astype(np.float64) * 2.0 ** -53          # [0, 1)
    return u1, u2


def normal_values(seed: int, name: str, numel: int, std: float, chunk: int = 1 << 22) -> np.ndarray:
    """float64 N(0, std) values of one tensor, element order = row-major."""
    key = tensor_key(seed, name)
    out = np.empty(numel, dtype=np.float64)
    for s in range(0, numel, chunk):
        n = min(chunk, numel - s)
        u1, u2 = _uniform_pairs(key, s, n)
        out[s:s + n] = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2) * std
    return out


def uniform_values(seed: int, name: str, numel: int, lo: float, hi: float) -> np.ndarray:
    key = tensor_key(seed, name)
    _, u = _uniform_pairs(key, 0, numel)
    return lo + (hi - lo) * u


def random_tensors(specs: Iterable[ParamSpec], seed: int, dtype: torch.dtype = torch.float32,
                   std: float = 0.02, norm_jitter: float = 0.0) -> Dict[str, torch.Tensor]:
    """CPU tensors for every declared parameter, in storage dtype ``dtype``."""
    out: Dict[str, torch.Tensor] = {}
    for s in specs:
        numel = int(np.prod(s.shape)) if s.shape else 1
        if s.kind == INT_TABLE:
            raise ValueError(f"no random rule for the integer table {s.name}")
        if s.init == "ones":
            v = np.ones(numel, dtype=np.float64)
            if norm_jitter:
                v = v + uniform_values(seed, s.name, numel, -norm_jitter, norm_jitter)
        else:
            v = normal_values(seed, s.name, numel, std)
        t = torch.from_numpy(v.astype(np.float32)).reshape(s.shape)
        store = torch.float32 if (s.kind == KEEP32 and dtype == torch.float32) else dtype
        out[s.name] = t.to(store)
    return out


def write_model_folder(folder: str, config, specs: Iterable[ParamSpec], seed: int,
                       dtype: torch.dtype = torch.float32, std: float = 0.02,
                       norm_jitter: float = 0.0) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config``; returns ``folder``."""
    os.makedirs(folder, exist_ok=True)
    specs = list(specs)
    tensors = random_tensors(specs, seed, dtype, std, norm_jitter)
    cfg = config.to_json()
    cfg["torch_dtype"] = {torch.float32: "float32", torch.bfloat16: "bfloat16"}[dtype]
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      [(s.name, tensors[s.name]) for s in specs],
                      metadata={"format": "pt", "seed": str(seed)})
    return folder
