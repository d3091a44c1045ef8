"""Norm wrappers and nGPT building blocks (reference: transformers/normalization.py:15-172)."""

from __future__ import annotations

import torch
from torch import nn
import torch.nn.functional as F

from halite_b200 import ops


class PreNormalization(nn.Module):
    def __init__(self, norm, module):
        super().__init__()
        self.norm = norm
        self.module = module

    def forward(self, input, *args, **kwargs):
        return self.module(self.norm(input), *args, **kwargs)

    def tp_plan(self):
        return {"norm": "sequence"}


class FusedPreNormalization(nn.Module):
    """norm(input + residual) feeding `module`; returns (module output, new residual). The add
    and the norm are one kernel on CUDA."""

    def __init__(self, norm, module, dropout=0):
        super().__init__()
        self.norm = norm
        self.module = module
        self.dropout = dropout

    def forward(self, input, residual=None, *args, **kwargs):
        if self.training and self.dropout > 0:
            input = F.dropout(input, self.dropout)
        if residual is None:
            residual = input
            normed = self.norm(input)
        else:
            normed, residual = self.norm(input, residual)
        out = self.module(normed, *args, **kwargs)
        if isinstance(out, tuple):
            return (out[0], residual, *out[1:])
        return out, residual


class FusedPostBlock(nn.Module):
    """Final norm(input + residual)."""

    def __init__(self, norm, dropout=0):
        super().__init__()
        self.norm = norm
        self.dropout = dropout

    def forward(self, input, residual=None):
        if residual is None:
            return self.norm(input)
        return self.norm(input, residual)[0]


class LinearLayer(nn.Sequential):
    """Linear followed by extra modules; initialisers address the linear at index 0."""


class NormalizedEmbedding(nn.Embedding):
    def forward(self, input):
        return F.normalize(super().forward(input), dim=-1)


class NormalizedLinear(nn.Linear):
    """Linear whose weight rows are kept on the unit sphere."""

    def forward(self, input):
        return ops.linear(input, F.normalize(self.weight, dim=-1), self.bias)


class Scale(nn.Module):
    """Learned per-channel scale stored at `init_scale` and applied as value * (init_value / init_scale)."""

    def __init__(self, dim, init_value=1.0, init_scale=1.0):
        super().__init__()
        self.init_value, self.init_scale = init_value, init_scale
        self.scale = nn.Parameter(torch.full((dim,), float(init_scale)))

    def init_weights(self):
        nn.init.constant_(self.scale, self.init_scale)

    def forward(self, input):
        return input * (self.scale * (self.init_value / self.init_scale)).to(input.dtype)


class L2Norm(nn.Module):
    def __init__(self, dim=-1, eps=1e-6):
        super().__init__()
        self.dim, self.eps = dim, eps

    def forward(self, input):
        return F.normalize(input.float(), dim=self.dim, eps=self.eps).type_as(input)
