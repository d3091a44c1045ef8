"""Reinforcement-learning reductions: generalized advantage estimation as one reverse scan.

Replaces the Python loop of T small kernels in the reference (projects/ppo/trainer.py:200-213).
"""

from __future__ import annotations

import torch

import halite_b200.ops as ops


def gae_reference(rewards, values, gamma, lam, mask=None):
    B, T = rewards.shape
    adv = torch.zeros_like(rewards)
    last = torch.zeros(B, dtype=rewards.dtype, device=rewards.device)
    next_v = torch.zeros_like(last)
    for t in reversed(range(T)):
        m = mask[:, t] if mask is not None else 1.0
        delta = rewards[:, t] + gamma * next_v - values[:, t]
        cur = delta + gamma * lam * last
        last = m * cur + (1 - m) * last
        next_v = m * values[:, t] + (1 - m) * next_v
        adv[:, t] = m * cur
    ret = adv + values * (mask if mask is not None else 1.0)
    return adv, ret


def gae(rewards, values, gamma=1.0, lam=0.95, mask=None):
    """advantages, returns = GAE(rewards, values); positions with mask == 0 are skipped."""
    if rewards.is_cuda and not ops.force_reference():
        m = mask.float().contiguous() if mask is not None else None
        return ops.ext().gae(rewards.float().contiguous(), values.float().contiguous(), m, gamma, lam)
    return gae_reference(rewards.float(), values.float(), gamma, lam,
                         mask.float() if mask is not None else None)
