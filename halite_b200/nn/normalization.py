"""Normalisation layers (reference: nn/normalization.py:13-57). On CUDA/bf16 the forward and
backward are the sm_100a RMSNorm kernels; elsewhere the eager fp32 definition."""

from __future__ import annotations

import torch
from torch import nn

from halite_b200 import ops


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, elementwise_affine=True, weight_init=None,
                 fast=False, weight_offset: float = 0.0):
        super().__init__()
        self.dim = dim
        self.eps = eps
        self.elementwise_affine = elementwise_affine
        self.weight_offset = weight_offset
        self.weight_init = weight_init
        if elementwise_affine:
            self.weight = nn.Parameter(torch.ones(dim))
        else:
            self.register_parameter("weight", None)
        self.fast = fast  # kept for config compatibility: the kernel path is chosen by device

    def init_weights(self):
        if not self.elementwise_affine:
            return
        if self.weight_init is not None:
            self.weight_init(self.weight)
        elif self.weight_offset:
            nn.init.zeros_(self.weight)
        else:
            nn.init.ones_(self.weight)

    def forward(self, input, residual=None):
        """With `residual`, returns (norm(input + residual), input + residual)."""
        return ops.rms_norm(input, self.weight, self.eps, residual, self.weight_offset)

    def extra_repr(self):
        return f"{self.dim}, eps={self.eps}, affine={self.elementwise_affine}"


class LayerNorm(nn.LayerNorm):
    def init_weights(self):
        if self.elementwise_affine:
            nn.init.ones_(self.weight)
            if self.bias is not None:
                nn.init.zeros_(self.bias)


class L2Norm(nn.Module):
    def __init__(self, dim=-1, eps=1e-6):
        super().__init__()
        self.dim, self.eps = dim, eps

    def forward(self, input):
        return torch.nn.functional.normalize(input.float(), dim=self.dim, eps=self.eps).type_as(input)
