"""The manager of engine B (reference: tokainfer/engine/manager.py): owns all scheduling state on
the host and keeps the worker `scheduling_steps_ahead` forwards busy without waiting for their
results.

Each scheduled forward contains one decode token for every running sequence plus prompt chunks
of the sequences being onboarded. New sequences are admitted only while the simulated KV usage
of everything running (with predicted completion lengths) stays within the pool. When decode
growth nevertheless runs out of blocks, the most recently started sequences are *bumped*: their
blocks are released and they re-enter the queue with prompt + generated tokens as the new
prompt. Results that arrive for finished or bumped sequences are dropped.
"""

from __future__ import annotations

import uuid
from collections import deque

from halite_b200.tokainfer.allocator import BatchIndexAllocator, BlockAllocator, NoSpaceException
from halite_b200.tokainfer.hydragen import group_for_hydragen, reorder_decoding_seqs_for_hydragen
from halite_b200.tokainfer.monitoring import StatsTracker, track_time
from halite_b200.tokainfer.scheduler import calc_prefill_per_forward, try_onboarding_seqs
from halite_b200.tokainfer.stopping_predictor import EarlyStoppingTracker
from halite_b200.tokainfer.types import ModelInput, SamplingParams, ScheduleDecision, Sequence


class Manager:
    def __init__(self, config, tokenizer, num_blocks, max_seqs, context_len, send_input, eos_token_ids=()):
        self.config, self.tokenizer = config, tokenizer
        self.context_len = config.max_seq_len or context_len
        self.send_input = send_input                  # callable(ModelInput)
        self.eos_token_ids = set(eos_token_ids)
        self.num_blocks = num_blocks
        self.allocator = BlockAllocator(num_blocks, config.page_size)
        self.batch_indices = BatchIndexAllocator(min(max_seqs, config.max_seqs_per_forward))
        self.predictor = EarlyStoppingTracker(
            config.early_stopping_buffer_size, config.early_stopping_initial_wait, config.early_stopping_init_mean,
            config.early_stopping_init_std, config.early_stopping_num_prediction_buckets,
            config.spec_allocation_std_buffer_scale)
        self.stats = StatsTracker(num_blocks)
        self.waiting: deque = deque()
        self.running: list = []               # admitted, in admission order
        self.by_index: dict = {}              # batch index -> Sequence
        self.pending_page_updates: list = []
        self.step_sent = 0
        self.step_done = 0
        self.inflight_steps: deque = deque()  # step ids sent, in order
        self.zombies: dict = {}               # batch index -> outstanding results of a released sequence
        self.finished: list = []

    # ------------------------------------------------------------------ intake
    def add_request(self, request_id, input_ids, sampling_params):
        sp = SamplingParams.coerce(sampling_params)
        ids = list(input_ids)[: self.context_len - 1]
        sp.max_new_tokens = max(0, min(sp.max_new_tokens, self.context_len - len(ids)))
        out = []
        for _ in range(max(sp.n, 1)):
            seq = Sequence(uuid.uuid4().hex, request_id, ids, sp)
            self.waiting.append(seq)
            out.append(seq)
        return out

    def cancel(self, request_ids):
        """Stop the named requests (reference: tokainfer/engine/manager.py cancellation commands): a
        waiting sequence never starts, a running one gives back its blocks now and the results of
        forwards already in flight for it are dropped when they arrive. Returns the sequences
        that were cancelled; they are reported with finish reason "cancelled" and the tokens
        received so far."""
        wanted = set(request_ids)
        hit = []
        for seq in [s for s in self.waiting if s.request_id in wanted]:
            self.waiting.remove(seq)
            seq.finished, seq.finish_reason = True, "cancelled"
            self.finished.append(seq)
            hit.append(seq)
        for seq in [s for s in self.running if s.request_id in wanted and not s.finished]:
            seq.finished, seq.finish_reason = True, "cancelled"
            self._release(seq, finished=False)
            self.finished.append(seq)
            hit.append(seq)
        return hit

    def idle(self):
        return not self.waiting and not self.running and not self.inflight_steps

    # ------------------------------------------------------------------ results
    def _predict(self, seq):
        if not self.config.track_early_stopping:
            return seq.sampling_params.max_new_tokens
        return self.predictor.predict_completion_length(seq)

    def process_output(self, out):
        assert self.inflight_steps and self.inflight_steps[0] == out.step_id, "results must arrive in order"
        self.inflight_steps.popleft()
        self.step_done = out.step_id
        done = []
        for row, tok, lp in zip(out.batch_indices, out.tokens, out.logprobs):
            if row in self.zombies:
                self.zombies[row] -= 1
                if self.zombies[row] == 0:
                    del self.zombies[row]
                    self.batch_indices.free_index(row)
                continue
            seq = self.by_index.get(row)
            if seq is None:
                continue
            seq.inflight -= 1
            if seq.finished:
                continue
            seq.output_ids.append(tok)
            seq.output_logprobs.append(lp)
            seq.tokens_received += 1
            reason = self._finish_reason(seq)
            if reason is not None:
                seq.finished, seq.finish_reason = True, reason
                done.append(seq)
        for seq in done:
            self._release(seq, finished=True)
        return done

    def _finish_reason(self, seq):
        sp, tok = seq.sampling_params, seq.output_ids[-1]
        if not sp.ignore_eos and tok in self.eos_token_ids:
            return "eos"
        if sp.stop_token_ids and tok in sp.stop_token_ids:
            return "stop_token"
        if sp.stop and self.tokenizer is not None:
            look = self.config.stop_string_num_token_lookback
            tail = self.tokenizer.decode(seq.output_ids[-look:])
            if any(s in tail for s in sp.stop):
                return "stop_string"
        if len(seq.output_ids) >= sp.max_new_tokens:
            return "length"
        return None

    def _release(self, seq, finished):
        """Give back blocks and (once nothing is in flight) the batch index."""
        if seq in self.running:
            self.running.remove(seq)
        # KV exists for the prompt and for every generated token that has been fed back in
        written = seq.prompt_scheduled + max(0, min(seq.decode_scheduled, len(seq.output_ids)) - (1 if finished else 0))
        tokens = (seq.input_ids + seq.output_ids)[:written]
        self.allocator.free_and_update(seq.id, seq.kv_indices, tokens)
        seq.kv_indices = []
        row = seq.batch_index
        self.by_index.pop(row, None)
        if seq.inflight > 0:
            self.zombies[row] = self.zombies.get(row, 0) + seq.inflight
        else:
            self.batch_indices.free_index(row)
        seq.batch_index = None
        if finished:
            self.predictor.add_finished_sequences([seq])
            self.stats.add_finished_seq()
            self.finished.append(seq)

    # ------------------------------------------------------------------ scheduling
    def _onboard(self):
        if not self.waiting or self.batch_indices.available() == 0:
            return
        cap = int(self.num_blocks * self.config.spec_allocation_target_kv_cache_utilization)
        limit = min(len(self.waiting), self.batch_indices.available())
        n = try_onboarding_seqs(self.running, list(self.waiting)[:limit], self.config.page_size, cap, self._predict,
                                prefill_rate=self.config.max_tokens_per_forward)
        if n == 0 and not self.running and self.waiting:
            n = 1                        # nothing else holds memory: the first must be allowed to try
        for _ in range(n):
            seq = self.waiting[0]
            try:
                cached, fresh = self.allocator.allocate_with_prefix_match(seq.id, seq.input_ids)
            except NoSpaceException:
                if not self.running and not self.inflight_steps:
                    # the pool is empty and the prompt still does not fit: it never will
                    self.waiting.popleft()
                    seq.finished, seq.finish_reason = True, "no_space"
                    self.finished.append(seq)
                    continue
                break
            self.waiting.popleft()
            seq.batch_index = self.batch_indices.allocate()
            seq.kv_indices = cached + fresh
            seq.cached_tokens = len(cached) * self.config.page_size
            seq.prompt_scheduled = seq.cached_tokens
            seq.decode_scheduled = 0
            seq.inflight = 0
            self.by_index[seq.batch_index] = seq
            self.pending_page_updates.append((seq.batch_index, 0, list(seq.kv_indices)))
            self.running.append(seq)

    def _bump(self, need_blocks):
        """Preempt the most recently admitted sequences until `need_blocks` are free."""
        while self.allocator.num_free_blocks() < need_blocks and len(self.running) > 1:
            seq = self.running[-1]
            self._release(seq, finished=False)
            seq.input_ids = seq.input_ids + seq.output_ids[: seq.tokens_received]
            seq.sampling_params.max_new_tokens -= seq.tokens_received
            seq.prior_output = getattr(seq, "prior_output", []) + seq.output_ids[: seq.tokens_received]
            seq.prior_logprobs = getattr(seq, "prior_logprobs", []) + seq.output_logprobs[: seq.tokens_received]
            seq.output_ids, seq.output_logprobs = [], []
            seq.tokens_received = seq.decode_scheduled = seq.prompt_scheduled = 0
            seq.bumped += 1
            self.stats.bumped += 1
            self.waiting.appendleft(seq)

    def make_decision(self):
        with track_time("schedule"):
            self._onboard()
            decoding = [s for s in self.running if s.prefill_done and not s.finished
                        and s.decode_scheduled < s.sampling_params.max_new_tokens - 1
                        # a decode step feeds back a token: it must exist here or be in flight
                        and s.decode_scheduled < s.tokens_received + s.inflight]
            decoding = decoding[: self.config.max_seqs_per_forward]
            need = sum(self.allocator.num_blocks_needed(s.kv_indices, s.total_scheduled_len() + 1) for s in decoding)
            if need > self.allocator.num_free_blocks():
                self._bump(need)
                decoding = [s for s in decoding if s in self.running]
            prefilling = calc_prefill_per_forward([s for s in self.running if not s.prefill_done], len(decoding),
                                                  self.config.max_tokens_per_forward,
                                                  self.config.prefill_round_up_multiple)
            prefilling = prefilling[: max(0, self.config.max_seqs_per_forward - len(decoding))]
            if self.config.use_hydragen and decoding:
                groups, _ = group_for_hydragen(decoding, self.config.page_size, self.config.hydragen_min_group_size,
                                               self.config.hydragen_min_prefix_len)
                decoding = reorder_decoding_seqs_for_hydragen(decoding, groups)
                grouped = sum(len(g.seq_ids) * len(g.block_ids) for g in groups)
                self.stats.add_hydragen_stats(grouped, sum(len(s.kv_indices) for s in decoding))
            if not decoding and not prefilling:
                return None
            self.step_sent += 1
            return ScheduleDecision(self.step_sent, decoding, prefilling)

    def apply_decision(self, d: ScheduleDecision):
        """Allocate what the forward writes, advance the counters and build the worker input."""
        rows, tokens, prefix, sample, temps, tps, tks, mps = [], [], [], [], [], [], [], []

        def add(seq, toks, pre, do_sample):
            sp = seq.sampling_params
            rows.append(seq.batch_index)
            tokens.append(toks)
            prefix.append(pre)
            sample.append(do_sample)
            temps.append(sp.temperature)
            tps.append(sp.top_p)
            tks.append(sp.top_k)
            mps.append(sp.min_p)

        for seq, n in d.prefilling:
            start = seq.prompt_scheduled
            last = start + n >= seq.prompt_len
            add(seq, seq.input_ids[start:start + n], start, last)
            seq.prompt_scheduled += n
            if last:
                seq.inflight += 1
        for seq in d.decoding:
            pos = seq.total_scheduled_len()
            new = self.allocator.allocate_up_to_length(seq.id, seq.kv_indices, pos + 1)
            if new:
                self.pending_page_updates.append((seq.batch_index, len(seq.kv_indices), new))
                seq.kv_indices.extend(new)
            known = seq.decode_scheduled < seq.tokens_received
            tok = [seq.output_ids[seq.decode_scheduled]] if known else None
            add(seq, tok, pos, True)
            seq.decode_scheduled += 1
            seq.inflight += 1
        inp = ModelInput(d.step_id, rows, self.pending_page_updates, tokens, prefix, sample, temps, tps, tks, mps)
        self.pending_page_updates = []
        self.inflight_steps.append(d.step_id)
        self.stats.add_decision(d, self.allocator.num_used_blocks())
        return inp

    def schedule_ahead(self):
        """Send forwards until `scheduling_steps_ahead` are outstanding or nothing is runnable."""
        sent = 0
        while len(self.inflight_steps) < self.config.scheduling_steps_ahead:
            d = self.make_decision()
            if d is None:
                break
            self.send_input(self.apply_decision(d))
            sent += 1
        self.stats.add_num_steps_to_schedule(sent)
        return sent

    def pop_finished(self):
        out, self.finished = self.finished, []
        return out
