"""The counter-based random numbers of the sampler.

``u = (mix64(mix64(seed ^ 0x6A09E667F3BCC909) ^ mix64(position * 4 + stream)) >> 11) * 2^-53``
with the splitmix64 finaliser as ``mix64`` (src/engine.cpp:12-16,35-38): a pure function
of (seed, position, stream), so a request draws the same numbers whether it ran alone, in
a crowd, or was preempted and recomputed.  ``position`` is the index the new token will
occupy (src/engine.cpp:473).  Streams: 0 sample; 1 accept, 2 residual and 3 draft belong to
speculative decoding (src/engine.cpp:31) and are unused here.
"""
from __future__ import annotations

_MASK = (1 << 64) - 1

STREAM_SAMPLE = 0
STREAM_ACCEPT = 1
STREAM_RESIDUAL = 2
STREAM_DRAFT = 3


def mix64(z: int) -> int:
    z &= _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def counter_uniform(seed: int, position: int, stream: int = STREAM_SAMPLE) -> float:
    z = mix64(mix64((seed ^ 0x6A09E667F3BCC909) & _MASK) ^ mix64((position * 4 + stream) & _MASK))
    return float(z >> 11) * 2.0 ** -53
