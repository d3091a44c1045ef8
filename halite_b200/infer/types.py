"""Request / result / configuration types of the in-process inference engine (reference:
transformers/infer/types.py:9-154, engine/batch.py:20-76)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, NamedTuple

import torch


class InferenceRequest(NamedTuple):
    id: str
    input_ids: list[int]
    sampling_params: dict[str, Any]


class InferenceResult:
    def __init__(self, id, input_ids=None, output_ids=None, output_logprobs=None, finish_reason=None,
                 num_cached_prompt_tokens=None):
        self.id = id
        self.input_ids = [] if input_ids is None else input_ids
        self.output_ids = [] if output_ids is None else output_ids
        self.output_logprobs = [] if output_logprobs is None else output_logprobs
        self.finish_reason = [] if finish_reason is None else finish_reason
        self.num_cached_prompt_tokens = [] if num_cached_prompt_tokens is None else num_cached_prompt_tokens

    def validate_lengths(self):
        n = len(self.output_ids)
        if not (n == len(self.output_logprobs) == len(self.finish_reason) == len(self.num_cached_prompt_tokens)):
            raise ValueError(
                "output_ids, output_logprobs, finish_reason and num_cached_prompt_tokens must have one "
                f"entry per sample, got {n}, {len(self.output_logprobs)}, {len(self.finish_reason)}, "
                f"{len(self.num_cached_prompt_tokens)}")

    def to_dict(self):
        return {"id": self.id, "input_ids": self.input_ids, "output_ids": self.output_ids,
                "output_logprobs": self.output_logprobs, "finish_reason": self.finish_reason,
                "num_cached_prompt_tokens": self.num_cached_prompt_tokens}

    def __repr__(self):
        outs = self.output_ids if len(self.output_ids) <= 2 else [self.output_ids[0], "...", self.output_ids[-1]]
        return f"InferenceResult(id={self.id}, n_input={len(self.input_ids)}, output_ids={outs})"


class SamplingParams:
    def __init__(self, max_new_tokens=128, min_new_tokens=0, temperature=1.0, top_p=1.0, top_k=-1,
                 min_p=0.0, n=1, stop=None, stop_token_ids=None, ignore_eos=False, seed=None):
        self.max_new_tokens = max_new_tokens
        self.min_new_tokens = min_new_tokens
        self.temperature = temperature
        self.top_p = top_p
        self.top_k = top_k if top_k != -1 else 1 << 30
        self.min_p = min_p
        self.n = n
        self.stop_strs = stop
        self.stop_token_ids = set(stop_token_ids) if stop_token_ids is not None else None
        self.ignore_eos = ignore_eos
        self.seed = seed
        self.stop_str_max_len = 0
        self.normalized = False
        if temperature is not None and temperature <= 0:
            # temperature 0 means greedy
            self.temperature = 1.0
            self.top_k = 1

    @property
    def greedy(self):
        return self.top_k <= 1

    def normalize(self, tokenizer):
        if self.normalized:
            return
        if self.stop_strs is None:
            self.stop_strs = []
        elif isinstance(self.stop_strs, str):
            self.stop_strs = [self.stop_strs]
        longest = 0
        for s in self.stop_strs:
            if tokenizer is not None:
                try:
                    ids = tokenizer.encode(s, add_special_tokens=False)
                except TypeError:
                    ids = tokenizer.encode(s)
                longest = max(longest, len(ids))
            else:
                longest = max(longest, len(s))
        self.stop_str_max_len = longest
        self.normalized = True


@dataclass
class ServerConfig:
    max_prefill_tokens: int = 16384          # new tokens per prefill batch
    chunked_prefill_size: int = 8192         # longer prompts are prefilled in chunks of this size
    default_init_new_token_ratio: float = 0.7
    default_min_new_token_ratio_factor: float = 0.14
    default_new_token_ratio_decay_steps: int = 600
    schedule_conservativeness: float = 1.0
    use_cudagraph: bool = False
    cudagraph_step: int = 16
    cudagraph_additonal_batch_size: tuple = ()
    cudagraph_max_batch_size: int = 512
    page_size: int = 16
    max_running_requests: int = 1024
    max_total_tokens: int | None = None      # overrides the memory-derived KV budget
    decode_steps_ahead: int = 8              # decode steps launched before the host reads tokens
    disable_radix_cache: bool = False
    radix_backend: str = "auto"            # "native" (C++ tree), "python", or "auto"
    # cleanup() keeps weights, KV pool and captured CUDA graphs on the device and load_state_dict()
    # copies new weights into place (same addresses), so rollouts after the first need no
    # allocation and no graph capture; for jobs where training and the engine fit side by side
    keep_resident: bool = False
    seed: int = 0


@dataclass
class ModelConfig:
    n_heads: int
    n_key_value_heads: int
    head_dim: int
    n_layers: int
    context_len: int
    tp_size: int = 1
    memory_fraction_static: float | None = None
    kv_cache_dtype: Any = "auto"
    gpu_id: int = 0
    device: Any = "cuda"
    distributed: bool = False
    vocab_size: int | None = None

    def __post_init__(self):
        if self.memory_fraction_static is None:
            table = [(16, 0.79), (8, 0.81), (4, 0.85), (2, 0.87)]
            self.memory_fraction_static = next((f for n, f in table if self.tp_size >= n), 0.88)
