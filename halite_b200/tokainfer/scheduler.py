"""Scheduling arithmetic of the manager (reference: tokainfer/engine/scheduler.py:16-682).

The question at every step: how many waiting sequences can start without the KV pool running
dry at some *future* step? Running sequences grow by one token per step, open a new page every
`page_size` tokens and give all pages back when they finish (at their predicted completion
length). `calc_block_usage_over_time` turns that into a piecewise-constant timeline;
`try_onboarding_seqs` finds, by doubling then bisection, the longest prefix of the waiting queue
whose addition keeps the peak under the pool size; `calc_prefill_per_forward` spreads the
admitted prompts' tokens over forwards within the per-forward token budget.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class BlockUsagePoint:
    step: int
    blocks: int


@dataclass
class BlockUsageOverTime:
    points: list            # [BlockUsagePoint], increasing step, usage holds until the next point
    peak: int


def _pages(tokens, page_size):
    return -(-tokens // page_size)


def calc_block_usage_over_time(seqs, page_size, predicted_lengths, horizon=None, prefill_rate=None):
    """`seqs`: objects with `prompt_len`, `total_scheduled_len()`; `predicted_lengths[i]`: expected
    generated tokens at finish. A sequence still prefilling reaches its full prompt after
    ceil(remaining / prefill_rate) steps (immediately when prefill_rate is None)."""
    events = {}                      # step -> delta blocks

    def add(step, delta):
        events[step] = events.get(step, 0) + delta

    for s, pred in zip(seqs, predicted_lengths):
        cur = s.total_scheduled_len()
        final = s.prompt_len + max(pred, 0)
        start_blocks = _pages(max(cur, 1), page_size)
        add(0, start_blocks)
        t0 = 0
        if cur < s.prompt_len:       # finish prefill first
            remaining = s.prompt_len - cur
            t0 = 1 if prefill_rate is None else -(-remaining // max(prefill_rate, 1))
            add(t0, _pages(s.prompt_len, page_size) - start_blocks)
            cur = s.prompt_len
        blocks = _pages(max(cur, 1), page_size)
        # one token per step from t0: a new page each time the length crosses a page boundary
        length = cur
        while True:
            next_boundary = blocks * page_size + 1          # length at which another page is needed
            if next_boundary > final:
                break
            add(t0 + (next_boundary - length), 1)
            blocks += 1
        end = t0 + max(final - length, 0) + 1
        add(end, -blocks)
    points, usage, peak = [], 0, 0
    for step in sorted(events):
        if horizon is not None and step > horizon:
            break
        usage += events[step]
        points.append(BlockUsagePoint(step, usage))
        peak = max(peak, usage)
    return BlockUsageOverTime(points, peak)


def simulate_blocks(counts_per_last_page_len, num_steps):
    """Pages opened over `num_steps` decode steps by sequences bucketed by how full their last
    page is: counts_per_last_page_len[r] sequences have r tokens in the last page (r = 0 means
    the last page is full)."""
    page_size = len(counts_per_last_page_len)
    total = 0
    for r, count in enumerate(counts_per_last_page_len):
        room = (page_size - r) % page_size           # tokens that still fit in the current page
        if num_steps > room:
            total += count * (-(-(num_steps - room) // page_size))
    return total


def try_onboarding_seqs(running, waiting, page_size, num_blocks, predict, existing_used=0, prefill_rate=None):
    """How many sequences from the head of `waiting` can be admitted. `predict(seq)` gives the
    expected completion length. `existing_used`: blocks held outside the simulated sequences
    (e.g. cached prefixes that cannot be evicted)."""
    if not waiting:
        return 0
    budget = num_blocks - existing_used

    def fits(k):
        seqs = list(running) + list(waiting[:k])
        usage = calc_block_usage_over_time(seqs, page_size, [predict(s) for s in seqs], prefill_rate=prefill_rate)
        return usage.peak <= budget

    if not fits(1):
        return 0
    lo, hi = 1, 2
    while hi <= len(waiting) and fits(hi):           # coarse: double
        lo, hi = hi, hi * 2
    hi = min(hi, len(waiting) + 1)
    while hi - lo > 1:                               # precise: bisect
        mid = (lo + hi) // 2
        if fits(mid):
            lo = mid
        else:
            hi = mid
    return lo


def calc_prefill_per_forward(prefilling, n_decoding, max_tokens_per_forward, round_up_multiple=16):
    """[(seq, n_tokens)] for the next forward: first-come first-served chunks of the prompts that
    still have tokens to schedule, within the token budget left after the decode tokens."""
    budget = max_tokens_per_forward - n_decoding
    out = []
    for s in prefilling:
        if budget <= 0:
            break
        remaining = s.prompt_len - s.prompt_scheduled
        if remaining <= 0:
            continue
        n = min(remaining, budget)
        if n < remaining and n > round_up_multiple:
            n = n // round_up_multiple * round_up_multiple    # keep chunk boundaries aligned
        out.append((s, n))
        budget -= n
    return out
