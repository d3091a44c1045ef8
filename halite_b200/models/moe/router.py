"""Top-k token-choice router with optional capacity limits and auxiliary losses
(reference: transformers/moe/router.py:12-182)."""

from __future__ import annotations

import math
from typing import Callable

import torch
from torch import nn
from torch.nn import functional as F

from halite_b200.models.initialize import init_weights
from halite_b200.models.moe import ops as moe_ops

DROPPED = torch.iinfo(torch.int64).max


def get_capacity(n_tokens, n_experts, capacity_factor, min_capacity=None):
    cap = math.ceil(n_tokens / n_experts * capacity_factor)
    return max(cap, min_capacity) if min_capacity is not None else cap


def top_k_softmax_with_capacity(logits, top_k, capacity_factor=None, pad_to_capacity=False, drop_policy="probs",
                                pre_softmax=False, deterministic=False):
    """-> (probs [T, k], expert index [T, k], tokens per expert before any dropping).

    `pre_softmax`: softmax over all experts, then top-k of the probabilities; otherwise top-k of
    the logits and a softmax over the selected k. With a capacity factor each expert keeps its
    `capacity` highest-probability (or earliest, `drop_policy="position"`) tokens; dropped slots
    get probability 0 and index `DROPPED`. `pad_to_capacity` returns expert-major
    [E, capacity] tensors instead."""
    n_tokens, n_experts = logits.shape
    if pre_softmax:
        scores = torch.softmax(logits, -1, dtype=torch.float32).type_as(logits)
        probs, top = torch.topk(scores, top_k, dim=1)
    else:
        if top_k == 1:
            raise ValueError("post-softmax routing needs top_k > 1")
        scores, top = torch.topk(logits, top_k, dim=1)
        probs = torch.softmax(scores, -1, dtype=torch.float32).type_as(logits)
    if capacity_factor is None:
        if deterministic:
            counts = moe_ops.bincount(top, n_experts)
        else:
            counts = torch.histc(top.float(), bins=n_experts, min=0, max=n_experts).long()
        return probs, top, counts
    capacity = get_capacity(n_tokens * top_k, n_experts, capacity_factor)
    gates = torch.zeros_like(logits).scatter(1, top, probs)
    chosen = torch.zeros_like(logits).scatter(1, top, 1)
    counts = chosen.sum(0)
    if drop_policy == "position":
        # earliest tokens first: rank by position among the tokens that chose the expert
        order = torch.where(chosen.bool(), -torch.arange(n_tokens, device=logits.device, dtype=logits.dtype)[:, None],
                            torch.full_like(logits, -float("inf")))
        _, cap_idx = torch.topk(order, min(capacity, n_tokens), dim=0, sorted=False)
        cap_probs = torch.gather(gates, 0, cap_idx)
    else:
        cap_probs, cap_idx = torch.topk(gates, min(capacity, n_tokens), dim=0, sorted=False)
    if pad_to_capacity:
        return cap_probs.T.contiguous(), cap_idx.T.contiguous(), counts
    kept = torch.zeros_like(logits).scatter(0, cap_idx, 1).bool() & chosen.bool()
    exceeded = ~torch.gather(kept, 1, top)
    return probs * ~exceeded, top.masked_fill(exceeded, DROPPED), counts


class TopKRouter(nn.Module):
    def __init__(self, in_features, n_experts, top_k, gate_init: Callable | None = None, z_loss=0.0,
                 load_balance_loss=0.0, capacity_factor=None, pad_to_capacity=False, drop_policy="probs",
                 pre_softmax=False, deterministic=False):
        super().__init__()
        self.n_experts, self.top_k = n_experts, top_k
        self.gate = nn.Linear(in_features, n_experts, bias=False)
        self.gate_init = gate_init
        self.z_loss, self.load_balance_loss = z_loss, load_balance_loss
        self.capacity_factor, self.pad_to_capacity = capacity_factor, pad_to_capacity
        self.drop_policy, self.pre_softmax, self.deterministic = drop_policy, pre_softmax, deterministic

    def init_weights(self):
        init_weights(self.gate, self.gate_init)

    def calc_z_loss(self, logits):
        if self.z_loss > 0 and self.training:
            return self.z_loss * torch.logsumexp(logits.float(), -1).square().mean()
        return None

    def calc_load_balance_loss(self, logits, tokens_per_expert, activation=None):
        """n_experts * <mean router probability, fraction of tokens> (1 when perfectly balanced)."""
        if not (self.load_balance_loss > 0 and self.training):
            return None
        probs = torch.softmax(logits, -1, dtype=torch.float32).sum(0)
        load = tokens_per_expert.to(probs)
        return self.load_balance_loss * self.n_experts * (F.normalize(probs, p=1, dim=0) * F.normalize(load, p=1, dim=0)).sum()

    def forward(self, input):
        # the gate is tiny (dim x n_experts): keep it in fp32 for stable routing decisions
        logits = F.linear(input.float(), self.gate.weight.float()).view(-1, self.n_experts)
        aux = {}
        z = self.calc_z_loss(logits)
        if z is not None:
            aux["router-z-loss"] = z
        probs, indices, counts = top_k_softmax_with_capacity(
            logits, self.top_k, self.capacity_factor, self.pad_to_capacity, self.drop_policy, self.pre_softmax,
            self.deterministic)
        lb = self.calc_load_balance_loss(logits, counts, probs)
        if lb is not None:
            aux["load-balance-loss"] = lb
        return probs.to(input.dtype), indices, aux
