"""Stateless pseudo-random permutation of [0, max_index] (reference: data/index_shuffle.py:4-59):
a balanced Feistel network over the next power of four, cycle-walked back into range. Any
position of the epoch can be computed directly, which is what makes the dataset resumable and
shardable without materialising a permutation."""

from __future__ import annotations

_MASK64 = (1 << 64) - 1


def _mix(x: int) -> int:
    x &= _MASK64
    x ^= x >> 33
    x = (x * 0xFF51AFD7ED558CCD) & _MASK64
    x ^= x >> 33
    x = (x * 0xC4CEB9FE1A85EC53) & _MASK64
    x ^= x >> 33
    return x


def index_shuffle(index: int, max_index: int, seed: int, rounds: int = 4) -> int:
    """Image of `index` under a seed-dependent bijection of {0, ..., max_index}."""
    if max_index <= 0:
        return 0
    bits = max(2, max_index.bit_length())
    bits += bits & 1
    half = bits // 2
    lo_mask = (1 << half) - 1
    x = index
    while True:
        left, right = x >> half, x & lo_mask
        for r in range(rounds):
            f = _mix((right << 20) ^ (seed * 0x9E3779B97F4A7C15) ^ (r * 0xD1B54A32D192ED03)) & lo_mask
            left, right = right, left ^ f
        x = (left << half) | right
        if x <= max_index:
            return x
