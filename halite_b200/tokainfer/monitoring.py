"""Throughput / utilisation statistics of the engine (reference: tokainfer/engine/monitoring.py)."""

from __future__ import annotations

import contextlib
import os
import statistics
import time
from collections import defaultdict

_TIMERS = defaultdict(list)
_ENABLED = os.environ.get("HALITE_TRACK_TIME", "0") == "1"


@contextlib.contextmanager
def track_time(key: str):
    """Accumulate wall time under `key` when HALITE_TRACK_TIME=1 (free otherwise)."""
    if not _ENABLED:
        yield
        return
    t0 = time.perf_counter()
    try:
        yield
    finally:
        _TIMERS[key].append(time.perf_counter() - t0)


def track_time_decorator(key=None):
    def deco(fn):
        name = key or fn.__qualname__

        def wrapper(*a, **kw):
            with track_time(name):
                return fn(*a, **kw)

        return wrapper

    return deco


def timers_summary():
    return {k: {"n": len(v), "total_s": sum(v), "mean_ms": 1e3 * sum(v) / len(v)} for k, v in _TIMERS.items() if v}


def maybe_stdev(values):
    return statistics.stdev(values) if len(values) > 1 else 0.0


class StatsTracker:
    def __init__(self, num_blocks=0):
        self.num_blocks = num_blocks
        self.reset()

    def reset(self):
        self.start = time.monotonic()
        self.prefill_tokens = self.decode_tokens = self.forwards = 0
        self.finished_seqs = self.finished_reqs = 0
        self.idle_time = 0.0
        self.kv_usage = []
        self.steps_scheduled = []
        self.hydragen_grouped = self.hydragen_total = 0
        self.bumped = 0

    def elapsed_time(self):
        return time.monotonic() - self.start

    def add_decision(self, decision, used_blocks=None):
        self.forwards += 1
        self.decode_tokens += len(decision.decoding)
        self.prefill_tokens += sum(n for _, n in decision.prefilling)
        if used_blocks is not None and self.num_blocks:
            self.kv_usage.append(used_blocks / self.num_blocks)

    def add_finished_seq(self):
        self.finished_seqs += 1

    def add_finished_req(self):
        self.finished_reqs += 1

    def add_manager_idle_time(self, seconds):
        self.idle_time += seconds

    def add_num_steps_to_schedule(self, n):
        self.steps_scheduled.append(n)

    def add_hydragen_stats(self, grouped, total):
        self.hydragen_grouped += grouped
        self.hydragen_total += total

    def calc_stats(self):
        t = max(self.elapsed_time(), 1e-9)
        toks = self.prefill_tokens + self.decode_tokens
        return {
            "prefill_tok_per_s": self.prefill_tokens / t, "decode_tok_per_s": self.decode_tokens / t,
            "tok_per_forward": toks / max(self.forwards, 1), "forward_per_s": self.forwards / t,
            "finished_seqs": self.finished_seqs, "finished_reqs": self.finished_reqs,
            "kv_usage_mean": sum(self.kv_usage) / len(self.kv_usage) if self.kv_usage else 0.0,
            "kv_usage_max": max(self.kv_usage) if self.kv_usage else 0.0,
            "manager_idle_frac": self.idle_time / t, "bumped_seqs": self.bumped,
            "hydragen_grouped_frac": self.hydragen_grouped / max(self.hydragen_total, 1),
        }


def format_value(value):
    if isinstance(value, float):
        return f"{value:,.2f}"
    return f"{value:,}"


def log_to_statsd(server_url, metrics, prefix="halite"):
    """Gauges to a statsd endpoint ("host:port") when the `statsd` package is present."""
    if not server_url:
        return False
    try:
        import statsd
    except ImportError:
        return False
    host, _, port = server_url.partition(":")
    client = statsd.StatsClient(host, int(port or 8125), prefix=prefix)
    for k, v in metrics.items():
        client.gauge(k, v)
    return True
