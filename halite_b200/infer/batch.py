"""Requests and batches of the continuous-batching scheduler (reference:
infer/engine/batch.py:11-547). Token positions map to KV slots through pages of
`page_size` tokens: slot = page_id * page_size + position % page_size."""

from __future__ import annotations

from dataclasses import dataclass
from enum import IntEnum, auto

import torch

from halite_b200.infer.types import SamplingParams


class ForwardMode(IntEnum):
    EXTEND = auto()
    DECODE = auto()

    def is_decode(self):
        return self == ForwardMode.DECODE


class FinishReason:
    def __init__(self, reason, is_error=False, length=None, matched=None):
        self.reason = reason
        self.is_error = is_error
        self.length = length
        self.matched = matched

    def __repr__(self):
        return f"FinishReason({self.reason})"


class Request:
    def __init__(self, id, input_ids, sampling_params: SamplingParams, eos_token_ids=None):
        self.id = id
        self.input_ids = list(input_ids)
        self.output_ids: list[int] = []
        self.output_logprobs: list[float] = []
        self.sampling_params = sampling_params
        self.eos_token_ids = eos_token_ids or set()
        self.finished_reason: FinishReason | None = None
        self.req_slot: int | None = None
        self.pages: list[int] = []
        self.n_prefix_pages = 0
        self.last_node = None
        self.n_computed = 0          # tokens whose KV is in the cache
        self.extend_len = 0          # tokens computed by the current prefill chunk
        self.is_chunked = False
        self.n_cached_prompt_tokens = 0
        self.decoded_text = ""
        self.n_retracted = 0
        self.pending_tokens = 0      # decode steps launched whose tokens the host has not read yet

    @property
    def fill_ids(self):
        """Tokens the cache must hold before the next sample: prompt plus anything generated
        before a retraction."""
        return self.input_ids + self.output_ids

    @property
    def seq_len(self):
        return len(self.input_ids) + len(self.output_ids)

    def finished(self):
        return self.finished_reason is not None

    def check_finished(self, tokenizer=None):
        if self.finished():
            return
        sp = self.sampling_params
        if len(self.output_ids) >= sp.max_new_tokens:
            self.finished_reason = FinishReason("length", length=sp.max_new_tokens)
            return
        if not self.output_ids or len(self.output_ids) < sp.min_new_tokens:
            return
        last = self.output_ids[-1]
        if not sp.ignore_eos and last in self.eos_token_ids:
            self.finished_reason = FinishReason("stop", matched=last)
            return
        if sp.stop_token_ids and last in sp.stop_token_ids:
            self.finished_reason = FinishReason("stop", matched=last)
            return
        if sp.stop_strs and tokenizer is not None:
            tail = tokenizer.decode(self.output_ids[-(sp.stop_str_max_len + 1):])
            for s in sp.stop_strs:
                if s in tail or s in self.decoded_text:
                    self.finished_reason = FinishReason("stop", matched=s)
                    return

    def reset_for_retract(self):
        self.req_slot = None
        self.pages = []
        self.n_prefix_pages = 0
        self.last_node = None
        self.n_computed = 0
        self.extend_len = 0
        self.is_chunked = False
        self.n_retracted += 1


@dataclass
class ForwardBatch:
    """Device tensors of one model forward."""

    mode: ForwardMode
    input_ids: torch.Tensor          # [T] int64
    positions: torch.Tensor          # [T] int64
    out_cache_loc: torch.Tensor      # [T] int64 flat KV slot of every new token
    req_slots: torch.Tensor          # [B] int32 rows of the page table
    seq_lens: torch.Tensor           # [B] int32 total tokens in cache after this forward
    extend_lens: torch.Tensor | None = None     # [B] int32 (EXTEND)
    prefix_lens: torch.Tensor | None = None     # [B] int32 (EXTEND)
    qo_indptr: torch.Tensor | None = None       # [B+1] int32 (EXTEND)
    page_table: torch.Tensor | None = None      # [max_reqs, max_pages] int32
    max_seq_len: int = 0
    max_extend_len: int = 0
    page_size: int = 16
    sample_indices: torch.Tensor | None = None  # [B] index of each request's last token in [T]
    # host copies (used by the CPU reference attention and by tests)
    seq_lens_cpu: list | None = None
    extend_lens_cpu: list | None = None

    @property
    def batch_size(self):
        return self.req_slots.shape[0]


@dataclass
class BatchSamplingParams:
    temperatures: torch.Tensor   # [B, 1] fp32
    top_ps: torch.Tensor
    top_ks: torch.Tensor
    min_ps: torch.Tensor
    is_all_greedy: bool
    need_min_p_sampling: bool
    need_top_k_top_p: bool

    @classmethod
    def from_requests(cls, requests, device):
        sps = [r.sampling_params for r in requests]
        f32 = lambda xs: torch.tensor(xs, dtype=torch.float32).to(device, non_blocking=True)
        return cls(
            temperatures=f32([sp.temperature for sp in sps]).view(-1, 1),
            top_ps=f32([sp.top_p for sp in sps]),
            top_ks=torch.tensor([min(sp.top_k, 1 << 30) for sp in sps], dtype=torch.int32).to(device, non_blocking=True),
            min_ps=f32([sp.min_p for sp in sps]),
            is_all_greedy=all(sp.top_k <= 1 for sp in sps),
            need_min_p_sampling=any(sp.min_p > 0 for sp in sps),
            need_top_k_top_p=any(sp.top_p < 1.0 or 1 < sp.top_k < (1 << 29) for sp in sps),
        )


class Batch:
    """A set of requests that run one forward together."""

    def __init__(self, requests, req_pool, kv_pool, radix_cache, device):
        self.requests = list(requests)
        self.req_pool = req_pool
        self.kv_pool = kv_pool
        self.radix_cache = radix_cache
        self.device = device
        self.mode = ForwardMode.EXTEND
        self.forward_batch: ForwardBatch | None = None
        self.sampling: BatchSamplingParams | None = None

    def __len__(self):
        return len(self.requests)

    def is_empty(self):
        return len(self.requests) == 0

    # ------------------------------------------------------------------ page allocation
    def _alloc_pages(self, n):
        if n == 0:
            return []
        pages = self.kv_pool.alloc(n)
        if pages is None:
            self.radix_cache.evict(n - self.kv_pool.available_pages())
            pages = self.kv_pool.alloc(n)
        return pages

    def _slots_for(self, req, start, end):
        ps = self.kv_pool.page_size
        return [req.pages[p // ps] * ps + p % ps for p in range(start, end)]

    # ------------------------------------------------------------------ prefill
    def prepare_for_extend(self):
        """Requests carry `n_computed` (cached prefix) and `extend_len` (new tokens this
        forward). Allocates request slots and pages, fills the page table, builds tensors."""
        self.mode = ForwardMode.EXTEND
        ps = self.kv_pool.page_size
        input_ids, positions, out_loc = [], [], []
        seq_lens, extend_lens, prefix_lens, slots = [], [], [], []
        for req in self.requests:
            if req.req_slot is None:
                got = self.req_pool.alloc(1)
                if got is None:
                    raise RuntimeError("out of request slots")
                req.req_slot = got[0]
                self.req_pool.write(req.req_slot, 0, req.pages)
            start, end = req.n_computed, req.n_computed + req.extend_len
            need = (end + ps - 1) // ps - len(req.pages)
            if need > 0:
                new = self._alloc_pages(need)
                if new is None:
                    raise RuntimeError("out of KV pages during prefill (scheduler budget violated)")
                self.req_pool.write(req.req_slot, len(req.pages), new)
                req.pages.extend(new)
            fill = req.fill_ids
            input_ids.extend(fill[start:end])
            positions.extend(range(start, end))
            out_loc.extend(self._slots_for(req, start, end))
            seq_lens.append(end)
            extend_lens.append(end - start)
            prefix_lens.append(start)
            slots.append(req.req_slot)
        dev = self.device
        i32 = lambda xs: torch.tensor(xs, dtype=torch.int32).to(dev, non_blocking=True)
        i64 = lambda xs: torch.tensor(xs, dtype=torch.int64).to(dev, non_blocking=True)
        indptr = [0]
        for e in extend_lens:
            indptr.append(indptr[-1] + e)
        self.forward_batch = ForwardBatch(
            mode=self.mode, input_ids=i64(input_ids), positions=i64(positions), out_cache_loc=i64(out_loc),
            req_slots=i32(slots), seq_lens=i32(seq_lens), extend_lens=i32(extend_lens),
            prefix_lens=i32(prefix_lens), qo_indptr=i32(indptr), page_table=self.req_pool.req_to_pages,
            max_seq_len=max(seq_lens), max_extend_len=max(extend_lens), page_size=ps,
            sample_indices=i64([x - 1 for x in indptr[1:]]), seq_lens_cpu=seq_lens,
            extend_lens_cpu=extend_lens)
        self.sampling = BatchSamplingParams.from_requests(self.requests, dev)
        return self.forward_batch

    # ------------------------------------------------------------------ decode
    def pages_needed_for_decode(self, steps=1):
        """New pages the next `steps` decode steps will open across the batch."""
        ps = self.kv_pool.page_size
        n = 0
        for req in self.requests:
            pos = req.seq_len + req.pending_tokens - 1    # position of the next token to write
            last = pos + steps - 1
            n += max(0, last // ps + 1 - len(req.pages))
        return n

    def check_decode_memory(self, steps=1):
        need = self.pages_needed_for_decode(steps)
        return self.kv_pool.available_pages() + self.radix_cache.evictable_pages >= need

    def alloc_for_decode(self, steps=1):
        """Open the pages that the next `steps` tokens of every request need."""
        ps = self.kv_pool.page_size
        for req in self.requests:
            pos = req.seq_len + req.pending_tokens - 1
            need = (pos + steps - 1) // ps + 1 - len(req.pages)
            if need > 0:
                new = self._alloc_pages(need)
                if new is None:
                    raise RuntimeError("out of KV pages during decode (retract first)")
                self.req_pool.write(req.req_slot, len(req.pages), new)
                req.pages.extend(new)

    def prepare_for_decode(self, last_tokens=None):
        """One new token per request. `last_tokens` (device tensor) feeds the previous step's
        samples without a host round trip; otherwise the host copies of output_ids are used."""
        self.mode = ForwardMode.DECODE
        ps = self.kv_pool.page_size
        self.alloc_for_decode(1)
        positions, out_loc, slots = [], [], []
        for req in self.requests:
            pos = req.seq_len + req.pending_tokens - 1
            positions.append(pos)
            out_loc.append(req.pages[pos // ps] * ps + pos % ps)
            slots.append(req.req_slot)
        dev = self.device
        i32 = lambda xs: torch.tensor(xs, dtype=torch.int32).to(dev, non_blocking=True)
        i64 = lambda xs: torch.tensor(xs, dtype=torch.int64).to(dev, non_blocking=True)
        if last_tokens is None:
            last_tokens = i64([r.fill_ids[-1] for r in self.requests])
        seq_lens = [p + 1 for p in positions]
        self.forward_batch = ForwardBatch(
            mode=self.mode, input_ids=last_tokens, positions=i64(positions), out_cache_loc=i64(out_loc),
            req_slots=i32(slots), seq_lens=i32(seq_lens), page_table=self.req_pool.req_to_pages,
            max_seq_len=max(seq_lens), max_extend_len=1, page_size=ps, seq_lens_cpu=seq_lens)
        if self.sampling is None or len(self.sampling.temperatures) != len(self.requests):
            self.sampling = BatchSamplingParams.from_requests(self.requests, dev)
        return self.forward_batch

    # ------------------------------------------------------------------ set operations
    def filter(self, keep_indices):
        self.requests = [self.requests[i] for i in keep_indices]
        self.sampling = None

    def merge(self, other: "Batch"):
        self.requests.extend(other.requests)
        self.sampling = None

    def retract_decode(self):
        """Free memory by sending requests back to the waiting queue: the ones with the fewest
        generated tokens (then the longest prompts) go first. Returns the retracted requests."""
        order = sorted(range(len(self.requests)),
                       key=lambda i: (len(self.requests[i].output_ids), -len(self.requests[i].input_ids)),
                       reverse=True)
        retracted = []
        while order and not self.check_decode_memory(1):
            if len(order) == 1:
                break
            idx = order.pop()
            req = self.requests[idx]
            retracted.append(req)
            self.kv_pool.free(req.pages[req.n_prefix_pages:])
            self.radix_cache.dec_lock_ref(req.last_node)
            self.req_pool.free(req.req_slot)
            req.reset_for_retract()
        keep = sorted(order)
        self.filter(keep)
        return retracted
