"""Masked statistics and loss aggregation for PPO (reference: projects/ppo/math_fn.py:6-129)."""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch.nn import functional as F


def masked_mean(values, masks):
    return torch.sum(values * masks) / masks.sum()


def masked_var(values, mean, masks):
    return ((values - mean) * masks).pow(2).sum() / masks.sum()


def dist_var_mean(tensor, group=None, mask=None):
    """(variance, mean) of `tensor` over every rank of `group` (two scalar all-reduces)."""
    if mask is not None:
        total, count = torch.sum(tensor * mask), mask.sum().to(tensor.dtype)
    else:
        total, count = tensor.sum(), torch.tensor(float(tensor.numel()), device=tensor.device)
    pack = torch.stack([total, count])
    if dist.is_initialized():
        dist.all_reduce(pack, group=group)
    mean = pack[0] / pack[1]
    dev = (tensor - mean) * (mask if mask is not None else 1.0)
    sq = dev.pow(2).sum()
    if dist.is_initialized():
        dist.all_reduce(sq, group=group)
    return sq / pack[1], mean


def whitening(tensor, shift_mean=True, eps=1e-8, mask=None):
    """(x - mean) / (std + eps), statistics over masked positions; with shift_mean=False the
    mean is added back (scale only)."""
    if mask is not None:
        mask = mask.to(tensor.dtype)
        mean = masked_mean(tensor, mask)
        var = masked_var(tensor, mean, mask)
    else:
        var, mean = torch.var_mean(tensor, correction=0)
    out = (tensor - mean) / (torch.sqrt(var) + eps)
    if not shift_mean:
        out = out + mean
    return out


def pad1d(tensor, pad, mode="constant", value=None):
    if mode == "constant":
        return F.pad(tensor, pad, mode, value)
    dtype = tensor.dtype
    t = tensor.to(torch.float32)
    if tensor.ndim < 2:
        return F.pad(t.unsqueeze(0), pad, mode=mode).squeeze(0).to(dtype)
    return F.pad(t, pad, mode=mode).to(dtype)


def left_pad(tensor, length, mode="constant", value=None):
    return pad1d(tensor, (length - tensor.shape[1], 0), mode=mode, value=value)


def right_pad(tensor, length, mode="constant", value=None):
    return pad1d(tensor, (0, length - tensor.shape[1]), mode=mode, value=value)


def get_attention_mask(sample, attention_mask, pad_token_id):
    mask = sample.not_equal(pad_token_id).to(torch.int64)
    mask[:, : attention_mask.shape[1]] = attention_mask
    return mask


def truncate_penalty(samples, rewards, eoc_token_id, penalty):
    """Samples that never produced the end-of-completion token receive `penalty` as reward."""
    unfinished = (samples == eoc_token_id).sum(-1) == 0
    rewards = rewards.clone()
    rewards[unfinished] = penalty
    return rewards


def aggregate_loss(loss, mask, mode, max_tokens=None):
    if mode == "token-mean":
        return masked_mean(loss, mask)
    if mode == "token-mean-seq-mean":
        return (torch.sum(loss * mask, -1) / mask.sum(-1).clamp(min=1)).mean()
    if mode == "token-sum":
        total = torch.sum(loss * mask) / loss.shape[0]
        return total / max_tokens if max_tokens is not None else total
    raise ValueError(f"unknown loss aggregation {mode!r}")
