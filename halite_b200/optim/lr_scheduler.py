"""Piecewise learning-rate schedules (reference: optim/lr_scheduler.py:9-208).

A `PhaseScheduler` holds a list of phases `(start, end, n_steps, shape)`; every `step()` writes
the interpolated rate into each optimizer param group. It is stateful (`state_dict`) so a
resumed run continues on the same curve.
"""

from __future__ import annotations

import math


def _linear(start, end, t):
    return start + (end - start) * t


def _cos(start, end, t):
    return end + (start - end) * (math.cos(math.pi * t) + 1) / 2


def _cospow(power):
    def fn(start, end, t):
        return end + (start - end) * ((math.cos(math.pi * t) + 1) / 2) ** power

    return fn


def _poly(power):
    def fn(start, end, t):
        return end + (start - end) * (1 - t) ** power

    return fn


def _tanh(lo=-4.0, hi=4.0):
    def fn(start, end, t):
        s = 0.5 * (1 + math.tanh(lo + (hi - lo) * t))
        return start + (end - start) * s

    return fn


def _exp(start, end, t):
    if start <= 0 or end <= 0:
        return _linear(start, end, t)
    return start * (end / start) ** t


def _flat(start, end, t):
    return start


def resolve_shape(shape):
    if callable(shape):
        return shape
    if isinstance(shape, (tuple, list)):
        name, *args = shape
        return {"cospow": _cospow, "poly": _poly, "tanh": _tanh}[name](*args)
    return {"linear": _linear, "lin": _linear, "cos": _cos, "exp": _exp, "flat": _flat,
            "poly": _poly(2), "tanh": _tanh(), "cospow": _cospow(2)}[shape]


class Phase:
    def __init__(self, start, end, n_iter, shape="linear"):
        self.start, self.end = start, end
        self.n_iter = max(int(n_iter), 0)
        self.fn = resolve_shape(shape)
        self.n = 0

    def step(self):
        t = self.n / self.n_iter if self.n_iter > 0 else 1.0
        self.n += 1
        return self.fn(self.start, self.end, min(t, 1.0))

    def reset(self):
        self.n = 0

    @property
    def is_done(self):
        return self.n >= self.n_iter


class PhaseScheduler:
    """phases: [(lr_start, lr_end, n_steps, shape)]. After the last phase the final value holds."""

    def __init__(self, optimizer, phases, cycle=False):
        self.optimizer = optimizer
        self.phases = [Phase(*p) for p in phases]
        self.cycle = cycle
        self.phase = 0
        self.lr = self.phases[0].start if self.phases else 0.0
        self.n_step = 0

    def __repr__(self):
        body = ", ".join(f"({p.start:.3g}->{p.end:.3g} x{p.n_iter})" for p in self.phases)
        return f"PhaseScheduler({body})"

    def step(self):
        self.n_step += 1
        while self.phase < len(self.phases) and self.phases[self.phase].is_done:
            self.phase += 1
            if self.phase >= len(self.phases) and self.cycle:
                for p in self.phases:
                    p.reset()
                self.phase = 0
        if self.phase < len(self.phases):
            self.lr = self.phases[self.phase].step()
        elif self.phases:
            self.lr = self.phases[-1].end
        for group in self.optimizer.param_groups:
            group["lr"] = self.lr * group.get("lr_mult", 1.0)
        return self.lr

    def get_last_lr(self):
        return [self.lr]

    def state_dict(self):
        return {"phase": self.phase, "lr": self.lr, "n_step": self.n_step,
                "counters": [p.n for p in self.phases]}

    def load_state_dict(self, state):
        self.phase = state["phase"]
        self.lr = state["lr"]
        self.n_step = state.get("n_step", 0)
        for p, n in zip(self.phases, state["counters"]):
            p.n = n


def cycle_scheduler(optimizer, lr, n_iter, initial_multiplier=4e-2, final_multiplier=1e-5, warmup=500,
                    plateau=0, decay=("linear", "cos")):
    """warm-up (lr * initial -> lr) / plateau / decay (lr -> lr * final) over `n_iter` steps.
    `warmup` and `plateau` given below 1 are fractions of `n_iter`."""
    if 0 < warmup < 1:
        warmup = int(n_iter * warmup)
    if 0 < plateau < 1:
        plateau = int(n_iter * plateau)
    warmup, plateau = int(warmup), int(plateau)
    phases = []
    if warmup > 0:
        phases.append((lr * initial_multiplier, lr, warmup, decay[0]))
    if plateau > 0:
        phases.append((lr, lr, plateau, "flat"))
    phases.append((lr, lr * final_multiplier, max(n_iter - warmup - plateau, 0), decay[1]))
    return PhaseScheduler(optimizer, phases)


def step_scheduler(optimizer, lr, milestones, gamma=0.1, warmup=0, warmup_multiplier=4e-2):
    phases = []
    prev = 0
    if warmup > 0:
        phases.append((lr * warmup_multiplier, lr, warmup, "linear"))
        prev = warmup
    cur = lr
    for m in milestones:
        phases.append((cur, cur, max(m - prev, 0), "flat"))
        prev = m
        cur = cur * gamma
    phases.append((cur, cur, 1, "flat"))
    return PhaseScheduler(optimizer, phases)


def exp_scheduler(optimizer, lr, n_iter, final_multiplier=1e-2, warmup=0, warmup_multiplier=4e-2):
    phases = []
    if warmup > 0:
        phases.append((lr * warmup_multiplier, lr, warmup, "linear"))
    phases.append((lr, lr * final_multiplier, max(n_iter - warmup, 0), "exp"))
    return PhaseScheduler(optimizer, phases)


def lr_finder(optimizer, lr_min, lr_max, n_iter, linear=False):
    return PhaseScheduler(optimizer, [(lr_min, lr_max, n_iter, "linear" if linear else "exp")])
