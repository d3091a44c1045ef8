"""Continuous-batching scheduler (reference: infer/engine/scheduler.py:18-400).

Policy: prefill first. Waiting requests are admitted by `PrefillAdder` while token budgets
last; the finished prefill joins the running (decode) batch. When KV pages run out during
decode the youngest requests are retracted to the waiting queue and the reservation ratio
`new_token_ratio` is raised; it decays while decoding goes well. Decode is issued several
steps ahead of the host (see `ModelRunner.decode_steps`).
"""

from __future__ import annotations



from halite_b200.infer.batch import Batch, ForwardMode, Request
from halite_b200.infer.radix_cache import RadixCache, make_radix_cache  # noqa: F401
from halite_b200.infer.schedule_policy import PrefillAdder
from halite_b200.infer.types import InferenceRequest, SamplingParams, ServerConfig
from halite_b200.logging import logger


class Scheduler:
    def __init__(self, model_runner, tokenizer, server_config: ServerConfig):
        self.model_runner = model_runner
        self.tokenizer = tokenizer
        self.server_config = server_config
        sc = server_config
        self.init_new_token_ratio = min(sc.default_init_new_token_ratio * sc.schedule_conservativeness, 1.0)
        self.min_new_token_ratio = min(self.init_new_token_ratio * sc.default_min_new_token_ratio_factor, 1.0)
        self.new_token_ratio_decay = (self.init_new_token_ratio - self.min_new_token_ratio) \
            / sc.default_new_token_ratio_decay_steps
        self.eos_token_ids = self._eos_ids(tokenizer)
        self.stats = {"prefill_tokens": 0, "cached_tokens": 0, "decode_tokens": 0, "retractions": 0,
                      "decode_steps": 0, "prefill_batches": 0}
        self.initialize()

    @staticmethod
    def _eos_ids(tokenizer):
        ids = set()
        if tokenizer is None:
            return ids
        for name in ("eos_id", "eos_token_id"):
            v = getattr(tokenizer, name, None)
            if isinstance(v, int):
                ids.add(v)
        extra = getattr(tokenizer, "additional_stop_token_ids", None)
        if extra:
            ids.update(extra)
        return ids

    def initialize(self):
        mr = self.model_runner
        self.req_pool = mr.req_pool
        self.kv_pool = mr.kv_pool
        self.device = mr.device
        self.tree_cache = make_radix_cache(self.server_config.page_size, self.kv_pool,
                                           disable=self.server_config.disable_radix_cache,
                                           backend=self.server_config.radix_backend)
        self.max_running_requests = mr.max_running_requests
        self.waiting_queue: list[Request] = []
        self.running_batch: Batch | None = None
        self.chunked_req: Request | None = None
        self.new_token_ratio = self.init_new_token_ratio
        self.last_tokens = None      # device tensor of the running batch's latest samples

    def cleanup(self):
        self.waiting_queue = []
        self.running_batch = None
        self.chunked_req = None
        self.tree_cache = None
        self.last_tokens = None
        # the pools belong to the model runner; a reference kept here would keep their memory
        self.req_pool = None
        self.kv_pool = None

    # ------------------------------------------------------------------ requests
    def build_batch_request(self, requests):
        out = []
        for i, req in enumerate(requests):
            if isinstance(req, Request):
                out.append(req)
                continue
            if isinstance(req, str):
                rid, ids, sp = i, self.tokenizer.encode(req), {}
            elif isinstance(req, InferenceRequest):
                rid, ids, sp = req.id, req.input_ids, req.sampling_params
            elif isinstance(req, dict):
                rid, ids, sp = req.get("id", i), req["input_ids"], req.get("sampling_params", {})
            else:
                rid, ids, sp = req
            if isinstance(ids, str):
                ids = self.tokenizer.encode(ids)
            if not isinstance(sp, SamplingParams):
                sp = SamplingParams(**(sp or {}))
            sp.normalize(self.tokenizer)
            out.append(Request(rid, list(ids), sp, self.eos_token_ids))
        return out

    def process_requests(self, requests):
        for r in requests:
            limit = self.model_runner.model_config.context_len
            if len(r.input_ids) >= limit:
                r.input_ids = r.input_ids[: limit - 1]
            r.sampling_params.max_new_tokens = max(
                0, min(r.sampling_params.max_new_tokens, limit - len(r.input_ids)))
            self.waiting_queue.append(r)

    # ------------------------------------------------------------------ main loop
    def infer_batch(self, requests):
        outputs = []
        finished, out = self.infer(requests)
        outputs.extend(out)
        while not finished:
            finished, out = self.infer([])
            outputs.extend(out)
        return outputs

    def infer(self, requests):
        """One scheduling step. Returns (idle, finished request tuples)."""
        self.process_requests(requests)
        batch = self.get_next_batch()
        if batch is None:
            self.check_memory()
            self.new_token_ratio = self.init_new_token_ratio
            return True, []
        if batch.mode.is_decode():
            return False, self.run_decode(batch)
        return False, self.run_prefill(batch)

    def check_memory(self):
        avail = self.kv_pool.available_pages() + self.tree_cache.evictable_pages
        if avail != self.kv_pool.num_pages:
            logger.warning(f"KV page leak: {avail} free or evictable of {self.kv_pool.num_pages}")
        if self.req_pool.available_size() != self.model_runner.max_requests:
            logger.warning("request slot leak: "
                           f"{self.req_pool.available_size()} free of {self.model_runner.max_requests}")

    def get_next_batch(self):
        new_batch = self.get_new_prefill_batch()
        if new_batch is not None:
            return new_batch
        if self.running_batch is None or self.running_batch.is_empty():
            self.running_batch = None
            return None
        return self.running_batch

    def get_new_prefill_batch(self):
        running = len(self.running_batch) if self.running_batch else 0
        if not self.waiting_queue and self.chunked_req is None:
            return None
        if running >= self.max_running_requests:
            return None
        sc = self.server_config
        adder = PrefillAdder(self.tree_cache, self.kv_pool, self.running_batch, self.new_token_ratio,
                             sc.max_prefill_tokens, sc.chunked_prefill_size, sc.page_size)
        if self.chunked_req is not None:
            # the unfinished prompt continues first
            self.tree_cache.dec_lock_ref(self.chunked_req.last_node)   # adder.add re-locks
            adder.add(self.chunked_req)
            if not adder.can_run:
                self.tree_cache.inc_lock_ref(self.chunked_req.last_node)
                return None
        for req in list(self.waiting_queue):
            if running + len(adder.can_run) >= self.max_running_requests:
                break
            if self.req_pool.available_size() <= len(adder.can_run):
                break
            self._match_prefix(req)
            if not adder.add(req):
                if req not in adder.can_run:
                    break
                # admitted as a partial chunk: nothing more fits in this batch
                break
        if not adder.can_run:
            return None
        chosen = set(id(r) for r in adder.can_run)
        self.waiting_queue = [r for r in self.waiting_queue if id(r) not in chosen]
        self.chunked_req = adder.chunked_req
        batch = Batch(adder.can_run, self.req_pool, self.kv_pool, self.tree_cache, self.device)
        batch.prepare_for_extend()
        return batch

    def _match_prefix(self, req):
        """Point a fresh (or retracted) request at its cached prefix."""
        if req.req_slot is not None:
            return
        fill = req.fill_ids
        # at least one token must be computed to obtain logits
        pages, node = self.tree_cache.match_prefix(fill[: len(fill) - 1])
        req.pages = list(pages)
        req.n_prefix_pages = len(pages)
        req.last_node = node
        req.n_computed = len(pages) * self.server_config.page_size
        if req.n_retracted == 0:
            req.n_cached_prompt_tokens = req.n_computed

    # ------------------------------------------------------------------ prefill
    def run_prefill(self, batch):
        self.stats["prefill_batches"] += 1
        self.stats["prefill_tokens"] += sum(r.extend_len for r in batch.requests)
        self.stats["cached_tokens"] += sum(r.n_computed for r in batch.requests if r.n_computed and r.extend_len)
        _, ids, logprobs = self.model_runner.forward_and_sample(batch)
        ids, logprobs = ids.tolist(), logprobs.tolist()
        decoding = []
        for i, req in enumerate(batch.requests):
            req.n_computed += req.extend_len
            if req.is_chunked:
                # more of the prompt to go: publish the full pages computed so far
                self.tree_cache.cache_unfinished_request(req, self.req_pool)
                continue
            if req.sampling_params.max_new_tokens > 0:
                req.output_ids.append(ids[i])
                req.output_logprobs.append(logprobs[i])
            req.check_finished(self.tokenizer)
            if req.sampling_params.max_new_tokens == 0 and not req.finished():
                from halite_b200.infer.batch import FinishReason

                req.finished_reason = FinishReason("length", length=0)
            if req.finished():
                self.tree_cache.cache_finished_request(req, self.req_pool)
            else:
                decoding.append(req)
        out = self._collect(batch.requests)
        if decoding:
            nb = Batch(decoding, self.req_pool, self.kv_pool, self.tree_cache, self.device)
            nb.mode = ForwardMode.DECODE
            if self.running_batch is None or self.running_batch.is_empty():
                self.running_batch = nb
            else:
                self.running_batch.merge(nb)
            self.last_tokens = None
        return out

    # ------------------------------------------------------------------ decode
    def _steps_ahead(self, batch):
        n = max(1, self.server_config.decode_steps_ahead)
        remaining = min(r.sampling_params.max_new_tokens - len(r.output_ids) for r in batch.requests)
        n = min(n, max(remaining, 1))
        if self.waiting_queue:
            n = min(n, 2)    # look for admission often while requests wait
        while n > 1 and not batch.check_decode_memory(n):
            n //= 2
        return n

    def run_decode(self, batch):
        if not batch.check_decode_memory(1):
            retracted = batch.retract_decode()
            self.stats["retractions"] += len(retracted)
            self.new_token_ratio = min(self.new_token_ratio + 0.1, 1.0)
            for r in retracted:
                r.pending_tokens = 0
            self.waiting_queue = retracted + self.waiting_queue
            self.last_tokens = None
            if batch.is_empty():
                self.running_batch = None
                return []
        else:
            self.new_token_ratio = max(self.new_token_ratio - self.new_token_ratio_decay,
                                       self.min_new_token_ratio)
        n = self._steps_ahead(batch)
        batch.alloc_for_decode(n)
        ids, logprobs = self.model_runner.decode_steps(batch, n, None)
        self.stats["decode_steps"] += n
        ids, logprobs = ids.tolist(), logprobs.tolist()     # one device -> host read per n steps
        keep = []
        for i, req in enumerate(batch.requests):
            req.pending_tokens = 0
            for s in range(n):
                req.output_ids.append(ids[s][i])
                req.output_logprobs.append(logprobs[s][i])
                self.stats["decode_tokens"] += 1
                req.check_finished(self.tokenizer)
                if req.finished():
                    break
            if req.finished():
                self.tree_cache.cache_finished_request(req, self.req_pool)
            else:
                keep.append(i)
        out = self._collect(batch.requests)
        batch.filter(keep)
        if batch.is_empty():
            self.running_batch = None
        return out

    def _collect(self, requests):
        return [(r.id, r.input_ids, r.output_ids, r.output_logprobs, r.finished_reason.reason,
                 r.n_cached_prompt_tokens) for r in requests if r.finished()]
