"""Admission of waiting requests into a prefill batch under token budgets (reference:
infer/engine/schedule_policy.py:5-112)."""

from __future__ import annotations


class PrefillAdder:
    """Budgets, all in tokens:

    * total: free + evictable KV capacity, minus what running requests are still expected to
      generate (their remaining `max_new_tokens` discounted by `new_token_ratio`);
    * input: new tokens in this prefill batch (`max_prefill_tokens`);
    * chunk: a prompt longer than the remaining chunk budget is prefilled partially.
    """

    RESERVE_CAP = 4096

    def __init__(self, radix_cache, kv_pool, running_batch, new_token_ratio, max_prefill_tokens,
                 chunked_prefill_size, page_size):
        self.radix_cache = radix_cache
        self.kv_pool = kv_pool
        self.page_size = page_size
        self.new_token_ratio = new_token_ratio
        self.rem_total = kv_pool.available_size() + radix_cache.evictable_size()
        self.rem_input = max_prefill_tokens
        self.rem_chunk = chunked_prefill_size
        self.can_run = []
        self.chunked_req = None
        if running_batch is not None:
            for r in running_batch.requests:
                left = r.sampling_params.max_new_tokens - len(r.output_ids)
                self.rem_total -= min(left, self.RESERVE_CAP) * new_token_ratio + page_size

    def _round_up(self, n):
        ps = self.page_size
        return (n + ps - 1) // ps * ps

    def add(self, req):
        """Try to admit `req` (already prefix-matched: req.n_computed, req.last_node).
        Returns False when the batch is full."""
        total_len = len(req.fill_ids)
        new_tokens = total_len - req.n_computed
        reserve = min(req.sampling_params.max_new_tokens - len(req.output_ids), self.RESERVE_CAP)
        need_total = self._round_up(new_tokens) + reserve * self.new_token_ratio + self.page_size
        if need_total > self.rem_total and self.can_run:
            return False
        if need_total > self.rem_total:
            # a lone request that cannot fit even an empty pool is admitted only if its
            # prompt fits; generation may later retract
            if self._round_up(new_tokens) > self.rem_total:
                return False
        if self.rem_input <= 0 or (self.rem_chunk is not None and self.rem_chunk <= 0):
            return False
        budget = self.rem_input if self.rem_chunk is None else min(self.rem_input, self.rem_chunk)
        if new_tokens <= budget:
            req.extend_len = new_tokens
            req.is_chunked = False
        else:
            if self.can_run and self.rem_chunk is None:
                return False
            # chunk boundary on a page boundary so the published prefix is whole pages
            take = budget // self.page_size * self.page_size
            if take <= 0:
                return False
            req.extend_len = take
            req.is_chunked = True
            self.chunked_req = req
        self.radix_cache.inc_lock_ref(req.last_node)
        self.can_run.append(req)
        self.rem_total -= self._round_up(req.extend_len) + reserve * self.new_token_ratio + self.page_size
        self.rem_input -= req.extend_len
        if self.rem_chunk is not None:
            self.rem_chunk -= req.extend_len
        return not req.is_chunked
