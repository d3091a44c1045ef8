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

    def forward(self, input):
        first, *rest = list(self)
        out = ops.linear(input, first.weight, first.bias) if type(first) is nn.Linear else first(input)
        for m in rest:
            out = m(out)
        return out


class NormalizedEmbedding(nn.Embedding):
    def forward(self, input):
        return F.normalize(super().forward(input), dim=-1)


class NormalizedLinear(nn.Linear):
    """Linear whose weight rows are kept on the unit sphere."""

    def forward(self, input):
        return ops.linear(input, F.normalize(self.weight, dim=-1), self.bias)


class Scale(nn.Module):
    """Learned per-channel scale for nGPT: the parameter is stored at magnitude `scale` and acts
    as `weight * init / scale` (times `rescale`), optionally through abs()."""

    def __init__(self, dim, init, scale, rescale=None, apply_abs=False):
        super().__init__()
        self.weight = nn.Parameter(torch.full((dim,), float(scale), dtype=torch.float32))
        self.init, self.scale, self.rescale, self.apply_abs = init, scale, rescale, apply_abs

    def init_weights(self):
        nn.init.constant_(self.weight, self.scale)

    def forward(self, input):
        factor = self.init / self.scale * (self.rescale if self.rescale is not None else 1.0)
        scale = self.weight * factor
        if self.apply_abs:
            scale = scale.abs()
        return input * scale.to(input.dtype)


class L2Norm(nn.Module):
    def __init__(self, dim=-1, eps=1e-6):
        super().__init__()
        self.dim, self.eps = dim, eps

    def forward(self, input):
        return F.normalize(input.float(), dim=self.dim, eps=self.eps).type_as(input)
