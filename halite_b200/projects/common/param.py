"""Sampling-parameter distributions for rollouts (reference: projects/common/param.py)."""

from __future__ import annotations


class Param:
    def sample(self, rng):
        raise NotImplementedError


class Uniform(Param):
    def __init__(self, low, high, integer=False):
        self.low, self.high, self.integer = low, high, integer

    def sample(self, rng):
        if self.integer:
            return rng.randint(int(self.low), int(self.high))
        return rng.uniform(self.low, self.high)


class Choice(Param):
    def __init__(self, *values, weights=None):
        self.values = list(values[0]) if len(values) == 1 and isinstance(values[0], (list, tuple)) else list(values)
        self.weights = weights

    def sample(self, rng):
        if self.weights is not None:
            return rng.choices(self.values, weights=self.weights, k=1)[0]
        return rng.choice(self.values)
