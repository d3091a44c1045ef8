"""Predicting how long completions will run, for speculative KV allocation
(reference: tokainfer/engine/stopping_predictor.py:12-400).

Finished sequences contribute the fraction `completion_len / max_new_tokens` to a ring buffer.
For a running sequence that has already produced a fraction f, the expected final fraction is
the conditional mean of buffered fractions >= f (plus `std_buffer_scale` conditional standard
deviations as a safety margin), tabulated over `num_buckets` values of f. Until enough
sequences have finished the tracker falls back to configured (or worst-case) values.
"""

from __future__ import annotations

import bisect
import math
from collections import deque


def calc_cumulative_mean_stds(sorted_vals):
    """For each i: mean and std of sorted_vals[i:] (suffix statistics), in one backward pass."""
    n = len(sorted_vals)
    means, stds = [0.0] * n, [0.0] * n
    s = sq = 0.0
    for i in range(n - 1, -1, -1):
        v = sorted_vals[i]
        s += v
        sq += v * v
        k = n - i
        m = s / k
        means[i] = m
        stds[i] = math.sqrt(max(sq / k - m * m, 0.0))
    return means, stds


class EarlyStoppingBuffer:
    def __init__(self, buffer_size: int):
        self.buffer_size = buffer_size
        self.initialize()

    def initialize(self):
        self.values = deque(maxlen=self.buffer_size)

    def cleanup(self):
        self.values = deque(maxlen=self.buffer_size)

    def __len__(self):
        return len(self.values)

    def empty(self):
        return not self.values

    def add(self, value: float):
        self.values.append(min(max(float(value), 0.0), 1.0))

    def mean(self):
        return sum(self.values) / len(self.values)

    def std(self):
        m = self.mean()
        return math.sqrt(sum((v - m) ** 2 for v in self.values) / len(self.values))


class PredictionMap:
    """Expected final fraction as a function of the fraction already produced."""

    def __init__(self, sorted_vals, num_buckets, std_buffer_scale):
        means, stds = calc_cumulative_mean_stds(sorted_vals)
        self.table = []
        for b in range(num_buckets + 1):
            f = b / num_buckets
            i = bisect.bisect_left(sorted_vals, f)
            if i >= len(sorted_vals):
                self.table.append(1.0)          # nobody seen running this long: assume the limit
            else:
                self.table.append(min(1.0, max(f, means[i] + std_buffer_scale * stds[i])))
        self.num_buckets = num_buckets

    def predict(self, frac: float) -> float:
        b = min(self.num_buckets, max(0, math.ceil(frac * self.num_buckets)))
        return max(frac, self.table[b])


class EarlyStoppingTracker:
    def __init__(self, buffer_size=2048, initial_wait=16, init_mean=None, init_std=None, num_buckets=1024,
                 std_buffer_scale=0.25):
        self.buffer = EarlyStoppingBuffer(buffer_size)
        self.initial_wait = initial_wait
        self.init_mean, self.init_std = init_mean, init_std
        self.num_buckets, self.std_buffer_scale = num_buckets, std_buffer_scale
        self._map = None
        self._dirty = True

    def initialize(self):
        self.buffer.initialize()
        self._map, self._dirty = None, True

    cleanup = initialize

    def add_finished_sequences(self, seqs):
        for s in seqs:
            limit = max(s.sampling_params.max_new_tokens, 1)
            self.buffer.add(len(s.output_ids) / limit)
        self._dirty = True

    def is_warmed_up(self):
        return len(self.buffer) >= self.initial_wait

    def buffer_mean(self):
        return self.buffer.mean() if not self.buffer.empty() else None

    def buffer_std(self):
        return self.buffer.std() if not self.buffer.empty() else None

    def make_prediction_map(self):
        if self._dirty or self._map is None:
            self._map = PredictionMap(sorted(self.buffer.values), self.num_buckets, self.std_buffer_scale)
            self._dirty = False
        return self._map

    def predict_completion_length(self, seq) -> int:
        """Expected number of generated tokens at finish (never below what exists already)."""
        limit = seq.sampling_params.max_new_tokens
        done = max(len(seq.output_ids), seq.decode_scheduled)
        if limit <= 0:
            return 0
        if self.is_warmed_up():
            frac = self.make_prediction_map().predict(done / limit)
        elif self.init_mean is not None:
            frac = min(1.0, self.init_mean + self.std_buffer_scale * (self.init_std or 0.0))
        else:
            frac = 1.0
        return min(limit, max(done + 1, math.ceil(frac * limit)))

    def predict_completion_lengths(self, seqs):
        return [self.predict_completion_length(s) for s in seqs]
