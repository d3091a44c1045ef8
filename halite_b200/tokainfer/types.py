"""Data carried between the server, the manager and the model worker
(reference: tokainfer/types.py:27-816)."""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any


@dataclass
class ServerConfig:
    page_size: int = 16
    kv_cache_num_tokens: int | None = None      # None: sized from free device memory
    memory_fraction: float = 0.85
    max_tokens_per_forward: int = 8192
    max_seqs_per_forward: int = 1024
    max_seq_len: int | None = None              # defaults to the model's context length
    scheduling_steps_ahead: int = 8
    prefill_round_up_multiple: int = 16
    stop_string_num_token_lookback: int = 5
    # speculative KV allocation from predicted completion lengths
    track_early_stopping: bool = True
    early_stopping_buffer_size: int = 2048
    early_stopping_num_prediction_buckets: int = 1024
    early_stopping_initial_wait: int = 16
    early_stopping_init_mean: float | None = None
    early_stopping_init_std: float | None = None
    spec_allocation_std_buffer_scale: float = 0.25
    spec_allocation_target_kv_cache_utilization: float = 1.0
    # shared-prefix grouping of decode sequences
    use_hydragen: bool = False
    hydragen_min_group_size: int = 32
    hydragen_min_prefix_len: int = 256
    use_cudagraphs: bool = True                 # decode-only forwards replay a graph per batch-size bucket
    placement: str = "inline"                   # "inline" (same process) or "process"
    dp_size: int = 1
    pp_size: int = 1
    tp_size: int = 1
    stats_report_seconds: float = 5.0
    statsd_server_url: str | None = None
    seed: int = 0


@dataclass
class SamplingParams:
    max_new_tokens: int = 128
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    n: int = 1
    stop: list | None = None
    stop_token_ids: list | None = None
    ignore_eos: bool = False

    @classmethod
    def coerce(cls, sp):
        if isinstance(sp, cls):
            return sp
        if isinstance(sp, dict):
            known = {k: v for k, v in sp.items() if k in cls.__dataclass_fields__}
        else:
            known = {k: getattr(sp, k) for k in cls.__dataclass_fields__ if hasattr(sp, k)}
        out = cls(**known)
        if isinstance(out.stop, str):
            out.stop = [out.stop]
        if out.temperature == 0:
            out.temperature, out.top_k = 1.0, 1
        return out


@dataclass
class Sequence:
    id: str
    request_id: Any
    input_ids: list
    sampling_params: SamplingParams
    output_ids: list = field(default_factory=list)
    output_logprobs: list = field(default_factory=list)
    kv_indices: list = field(default_factory=list)       # page ids, in order
    batch_index: int | None = None
    prompt_scheduled: int = 0         # prompt tokens already sent to the worker (incl. cached prefix)
    cached_tokens: int = 0
    decode_scheduled: int = 0         # decode steps sent to the worker
    tokens_received: int = 0          # sampled tokens that have come back
    inflight: int = 0                 # forwards sent whose sampled token has not come back
    finished: bool = False
    finish_reason: str | None = None
    expected_completion_length: int | None = None
    arrival: float = field(default_factory=time.monotonic)
    bumped: int = 0

    @property
    def prompt_len(self):
        return len(self.input_ids)

    @property
    def prefill_done(self):
        return self.prompt_scheduled >= self.prompt_len

    def total_scheduled_len(self):
        """Tokens whose KV has been (or is scheduled to be) written."""
        return self.prompt_scheduled + self.decode_scheduled

    def max_total_len(self):
        return self.prompt_len + self.sampling_params.max_new_tokens


@dataclass
class ScheduleDecision:
    step_id: int
    decoding: list            # [Sequence]
    prefilling: list          # [(Sequence, n_tokens)]

    def num_tokens(self):
        return len(self.decoding) + sum(n for _, n in self.prefilling)

    def num_seqs(self):
        return len(self.decoding) + len(self.prefilling)


@dataclass
class ModelInput:
    """One forward. Entries are ordered prefill first, then decode."""

    step_id: int
    batch_indices: list        # row of the worker's page table per entry
    page_updates: list         # [(batch_index, first_page_slot, [page ids])]
    tokens: list               # per entry: list of token ids, or None = feed the last sampled token
    prefix_lens: list          # tokens already cached per entry
    sample: list               # per entry: sample a token after this forward?
    temperatures: list
    top_ps: list
    top_ks: list
    min_ps: list


@dataclass
class ModelOutput:
    step_id: int
    batch_indices: list
    tokens: list
    logprobs: list


@dataclass
class Command:
    kind: str                  # "cleanup" | "initialize" | "load_state_dict" | "shutdown"
    payload: Any = None
