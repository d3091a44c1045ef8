"""Rollout data model and the generate -> reward pipeline (reference:
projects/common/rollout.py:16-299).

A `Rollout` is one prompt (later: one sampled completion of it) with free-form `state`.
`RequestBuilder` turns a data batch into rollouts, `RolloutGenerator` runs them through the
inference engine, expands the n samples, runs per-rollout preprocessors (e.g. detokenisation)
and lets the `RewardRegistry` attach rewards.
"""

from __future__ import annotations

import dataclasses
import uuid
from dataclasses import dataclass, field
from random import Random
from typing import Any, NamedTuple

import torch

from halite_b200.infer.types import InferenceRequest
from halite_b200.projects.common.param import Param

_RESERVED = ("id", "input_ids", "output_ids", "output_logprobs", "type", "rewards", "rewards_dict",
             "sampling_params", "state")


class Response(NamedTuple):
    id: str
    responses: list
    response_logprobs: list | None = None


@dataclass
class Rollout:
    id: str
    input_ids: list
    output_ids: list | None = None
    output_logprobs: list | None = None
    type: str | None = None
    rewards: Any = None
    rewards_dict: dict | None = None
    sampling_params: dict = field(default_factory=dict)
    state: dict = field(default_factory=dict)

    def to_inference_request(self) -> InferenceRequest:
        return InferenceRequest(id=self.id, input_ids=self.input_ids, sampling_params=self.sampling_params)

    def has_field(self, key):
        return key in _RESERVED or key in self.state

    def get_field(self, key):
        return getattr(self, key) if key in _RESERVED else self.state[key]

    def set_field(self, key, value):
        if key in _RESERVED:
            raise AttributeError(f"`{key}` is a reserved rollout field; store extra data under another name")
        self.state[key] = value

    def copy(self):
        return dataclasses.replace(self, state=dict(self.state))


class Handler:
    """One reward function: `fn(*[list of field values per arg])` -> tensor [n] or [n, T].
    `targets` restricts it to rollout types; other rollouts receive `reward_padding`."""

    def __init__(self, name, fn, args=("output_texts",), targets="*", preprocess=None, reward_padding=0):
        self.name = name
        self.fn = fn
        self.args = args
        self.targets = targets
        self.preprocess = preprocess
        self.reward_padding = reward_padding

    def applies_to(self, rollout):
        return self.targets == "*" or rollout.type in self.targets


class RewardRegistry:
    def __init__(self, *handlers, postprocess=None):
        self.handlers = list(handlers)
        self.postprocess = postprocess
        if len(self.handlers) > 1 and postprocess is None:
            raise ValueError("several reward handlers need a `postprocess` that combines them")

    def __getitem__(self, i):
        return self.handlers[i]

    def __call__(self, rollouts):
        table = {}
        for h in self.handlers:
            rows = [i for i, r in enumerate(rollouts) if h.applies_to(r)]
            columns = [[rollouts[i].get_field(k) for i in rows] for k in h.args]
            if h.preprocess is not None:
                columns = h.preprocess(*columns)
            values = torch.as_tensor(h.fn(*columns))
            shape = (len(rollouts),) + tuple(values.shape[1:])
            full = values.new_full(shape, h.reward_padding)
            if rows:
                full[torch.tensor(rows)] = values
            table[h.name] = full
        if self.postprocess is not None:
            rewards, table = self.postprocess(table, rollouts)
        else:
            rewards = next(iter(table.values()))
        for i, r in enumerate(rollouts):
            r.rewards = rewards[i]
            r.rewards_dict = {k: v[i] for k, v in table.items()}
        return rollouts


class RequestBuilder:
    def __init__(self, prompt_key, sampling_params, tokenizer=None, type=None, type_key=None,
                 meta_maps=None, seed=None):
        if (type is None) == (type_key is None):
            raise ValueError("give exactly one of `type` and `type_key`")
        self.prompt_key = prompt_key
        self.sampling_params = sampling_params
        self.tokenizer = tokenizer
        self.type = type
        self.type_key = type_key
        self.meta_maps = meta_maps or {}
        self.random = Random(seed)

    def sample_sampling_params(self):
        return {k: (v.sample(self.random) if isinstance(v, Param) else v)
                for k, v in self.sampling_params.items()}

    def __call__(self, batch):
        keys = {self.prompt_key, *self.meta_maps.values()}
        if self.type_key is not None:
            keys.add(self.type_key)
        records = batch.unbind(keys)
        prompts = [r[self.prompt_key] for r in records]
        if self.tokenizer is not None:
            if hasattr(self.tokenizer, "encode_batch"):
                prompts = self.tokenizer.encode_batch(prompts)
            else:
                prompts = [self.tokenizer.encode(p) for p in prompts]
        out = []
        for prompt, rec in zip(prompts, records):
            out.append(Rollout(
                id=uuid.uuid4().hex, input_ids=list(prompt),
                type=self.type if self.type is not None else rec[self.type_key],
                sampling_params=self.sample_sampling_params(),
                state={k: rec[v] for k, v in self.meta_maps.items()}))
        return out


class RolloutGenerator:
    def __init__(self, inference_engine, reward_registry, preprocessors=None, finish_condition=None):
        self.inference_engine = inference_engine
        self.reward_registry = reward_registry
        self.preprocessors = list(preprocessors or [])
        self.finish_condition = finish_condition

    def initialize(self):
        self.inference_engine.initialize()

    def cleanup(self):
        self.inference_engine.cleanup()

    def load_state_dict(self, state_dict, assign=True):
        self.inference_engine.load_state_dict(state_dict, assign=assign)

    def load_from_model(self, model):
        """Weight hand-over from a (sharded) training model; engines that have a fused reshard
        path use it, the others go through the state dict."""
        if hasattr(self.inference_engine, "load_from_model"):
            self.inference_engine.load_from_model(model)
        else:
            self.inference_engine.load_state_dict(model.state_dict())

    def generate(self, rollouts):
        results = self.inference_engine.infer_batch([r.to_inference_request() for r in rollouts])
        by_id = {res.id: res for res in results}
        ids = [by_id[r.id].output_ids for r in rollouts]
        lps = [by_id[r.id].output_logprobs for r in rollouts]
        return self.build_rollout(rollouts, ids, lps if all(l for l in lps) else None)

    def build_rollout(self, rollouts, output_ids, output_logprobs=None):
        expanded = []
        for i, (r, samples) in enumerate(zip(rollouts, output_ids)):
            for j, sample in enumerate(samples):
                c = r.copy()
                c.output_ids = sample
                if output_logprobs is not None:
                    c.output_logprobs = output_logprobs[i][j]
                for fn in self.preprocessors:
                    c = fn(c)
                expanded.append(c)
        return self.reward_registry(expanded)
