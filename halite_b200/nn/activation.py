"""Activation modules (reference: nn/activation.py:6-95): gated units operate on a tensor
whose last dimension holds the two halves side by side."""

from __future__ import annotations


import torch
from torch import nn
import torch.nn.functional as F

from halite_b200.ops.activation import gated_act_packed


class SwiGLU(nn.Module):
    """silu(left half) * right half."""

    def forward(self, input):
        return gated_act_packed(input, "silu", gate_first=True)


class GEGLU(nn.Module):
    def __init__(self, approximate="none"):
        super().__init__()
        self.approximate = approximate

    def forward(self, input):
        if self.approximate == "tanh":
            return gated_act_packed(input, "gelu_tanh", gate_first=True)
        left, right = input.chunk(2, -1)
        return F.gelu(left, approximate=self.approximate) * right


class _BloomGELUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        return x * 0.5 * (1.0 + torch.tanh(0.79788456 * x * (1 + 0.044715 * x * x)))

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        t = torch.tanh(0.79788456 * x * (1 + 0.044715 * x * x))
        ff = 0.5 * x * ((1 - t * t) * (0.79788456 + 0.1070322243 * x * x)) + 0.5 * (1 + t)
        return ff * g


class BloomGELU(nn.Module):
    """tanh-approximated GELU with a hand-written backward (no saved intermediates)."""

    def forward(self, input):
        if self.training:
            return _BloomGELUFn.apply(input)
        return input * 0.5 * (1.0 + torch.tanh(0.79788456 * input * (1 + 0.044715 * input * input)))
