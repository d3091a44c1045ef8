"""Weight initialisers with explicit fan dimensions (reference: nn/init.py:7-75)."""

from __future__ import annotations

import math

import torch
from torch import nn


def _fan(tensor, fan_in_dim, fan_out_dim):
    shape = tensor.shape
    receptive = 1
    if tensor.dim() > 2:
        for i, s in enumerate(shape):
            if i not in (fan_in_dim % tensor.dim(), fan_out_dim % tensor.dim()):
                receptive *= s
    return shape[fan_in_dim] * receptive, shape[fan_out_dim] * receptive


@torch.no_grad()
def kaiming_normal_(tensor, a=0, mode="fan_in", nonlinearity="linear", fan_in_dim=1, fan_out_dim=0,
                    scale=1.0, truncate=None):
    """N(0, gain^2 / fan) with the fan read from the named dimensions; optional truncation at
    `truncate` standard deviations."""
    fan_in, fan_out = _fan(tensor, fan_in_dim, fan_out_dim)
    fan = fan_in if mode == "fan_in" else fan_out
    gain = nn.init.calculate_gain(nonlinearity, a)
    std = gain / math.sqrt(fan) * scale
    if truncate is not None:
        return nn.init.trunc_normal_(tensor, 0.0, std, -truncate * std, truncate * std)
    return tensor.normal_(0, std)


@torch.no_grad()
def kaiming_linear_(tensor, **kwargs):
    return kaiming_normal_(tensor, nonlinearity="linear", **kwargs)


@torch.no_grad()
def normal_(tensor, std=0.02, mean=0.0):
    return tensor.normal_(mean, std)
