"""Batch containers of the PPO trainer (reference: projects/ppo/types.py:10-120)."""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import fields
from typing import NamedTuple

import torch


def _split_fields(items, n_chunk, batch_size):
    cols = {}
    for k, v in items:
        if isinstance(v, torch.Tensor) and v.dim() > 0:
            cols[k] = v.chunk(n_chunk, dim=0)
        elif hasattr(v, "split") and not isinstance(v, (str, torch.Tensor)):
            cols[k] = v.split(batch_size)
        elif isinstance(v, Sequence) and not isinstance(v, str):
            cols[k] = [v[i:i + batch_size] for i in range(0, len(v), batch_size)]
        else:
            cols[k] = [v] * n_chunk
    return [{k: c[i] for k, c in cols.items()} for i in range(n_chunk)]


class Batch(NamedTuple):
    input_ids: torch.Tensor          # [B, P + R]: prompts left-padded, responses right-padded
    response_ids: torch.Tensor       # [B, R], pad_id beyond each response
    attention_mask: torch.Tensor
    position_ids: torch.Tensor
    rewards: torch.Tensor            # [B, R] token rewards
    ids: torch.Tensor                # [B] prompt group id
    prompt_len: torch.Tensor
    response_len: torch.Tensor
    temperatures: torch.Tensor | float
    response_logprobs: torch.Tensor | None = None

    def split(self, batch_size):
        n = self.input_ids.shape[0]
        if n % batch_size:
            raise ValueError(f"batch size {batch_size} does not divide {n} rows")
        n_chunk = max(1, n // batch_size)
        return [Batch(**d) for d in _split_fields(self._asdict().items(), n_chunk, batch_size)]


class RolloutBatch(NamedTuple):
    rollouts: list
    rewards: torch.Tensor
    batch: Batch | None = None
    returns: torch.Tensor | None = None
    advantages: torch.Tensor | None = None
    actor_log_probs: torch.Tensor | None = None
    actor_entropy: torch.Tensor | None = None
    inference_log_probs: torch.Tensor | None = None
    values: torch.Tensor | None = None

    def split(self, batch_size):
        n = self.rewards.shape[0]
        if n % batch_size:
            raise ValueError(f"batch size {batch_size} does not divide {n} rows")
        return [RolloutBatch(**d) for d in _split_fields(self._asdict().items(), n // batch_size, batch_size)]


class CriticMetrics(NamedTuple):
    rewards_mean: torch.Tensor
    advantage_mean: torch.Tensor
    advantage_var: torch.Tensor
    return_mean: torch.Tensor
    return_var: torch.Tensor


class ActorLossMixin:
    """Dataclass mixin: `metric_dict()` names every field `actor/<field>` and the critic
    statistics `critic/<field>`."""

    def metric_dict(self):
        out = {"actor/" + f.name: getattr(self, f.name) for f in fields(self) if f.name != "critic_metrics"}
        out.update({"critic/" + k: v for k, v in self.critic_metrics._asdict().items()})
        return out
