"""Greedy and temperature sampling.

The reference samples with exactly two rules (src/engine.cpp:40-80; README.md:207 lists
top-k / top-p as not implemented): the first index of the maximum when
``temperature <= 0``, else the inverse CDF of ``exp((l - max) / T)`` with 64-bit sums in
vocabulary order at the uniform number keyed by (seed, position).  On the device this is
one kernel over the step's wanted logits rows (csrc/common.cu); :func:`sample_row_host` is
its host twin for tests and for callers that hold logits on the host.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .rng import counter_uniform


@dataclass
class SamplingParams:
    """Per-request sampling options, named as in the reference (src/engine.h:26-31)."""
    temperature: float = 0.0   # 0 means greedy
    seed: int = 0
    max_new_tokens: int = 32
    ignore_eos: bool = False


def argmax_row_host(logits) -> int:
    l = np.asarray(logits)
    return int(np.flatnonzero(l == l.max())[0])


def sample_row_host(logits, temperature: float, u: float) -> int:
    l = np.asarray(logits, dtype=np.float32)
    if temperature <= 0:
        return argmax_row_host(l)
    w = np.exp(((l - l.max()) / np.float32(temperature)).astype(np.float32)).astype(np.float32)
    cum = np.cumsum(w.astype(np.float64))
    hit = np.flatnonzero((cum > u * cum[-1]) & (w > 0))
    return int(hit[0]) if len(hit) else int(np.flatnonzero(w > 0)[-1])


def uniform_for(params: SamplingParams, position: int) -> float:
    return counter_uniform(params.seed, position)
