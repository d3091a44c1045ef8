"""Transformer blocks (reference: transformers/block.py:10-165)."""

from __future__ import annotations

from typing import Any

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint


def _run_ff(block, module, x):
    """The feed-forward half of a block, recomputed in backward when the block's `checkpoint_ff`
    flag is set (selective activation checkpointing, per-op form)."""
    if getattr(block, "checkpoint_ff", False) and block.training and torch.is_grad_enabled() and x.requires_grad:
        return checkpoint(module, x, use_reentrant=False)
    return module(x)


class ResidualBlock(nn.Module):
    """input + dropout(post_norm(module(pre_norm(input))))."""

    def __init__(self, pre_norm, module, post_norm=None, dropout=0):
        super().__init__()
        self.pre_norm = pre_norm
        self.module = module
        self.post_norm = post_norm
        self.dropout = nn.Dropout(dropout)

    def forward(self, input, *args, **kwargs):
        out = input
        if self.pre_norm is not None:
            out = self.pre_norm(input)
        out = self.module(out, *args, **kwargs)
        rest = None
        if isinstance(out, tuple):
            out, *rest = out
        if self.post_norm is not None:
            out = self.post_norm(out)
        out = input + self.dropout(out)
        if rest is not None:
            return (out, *rest)
        return out

    def tp_plan(self):
        plan = {}
        if self.pre_norm is not None:
            plan["pre_norm"] = "sequence"
        if self.post_norm is not None:
            plan["post_norm"] = "sequence"
        return plan


class TransformerEncoderBlock(nn.Module):
    """self_attention then ff, each usually wrapped in a ResidualBlock. Returns
    (out, residual, next_cache, aux)."""

    def __init__(self, self_attention, ff):
        super().__init__()
        self.self_attention = self_attention
        self.ff = ff

    def forward(self, input, residual=None, attention_mask=None, attention_bias=None, pos_emb: Any = None,
                cache: Any = None, use_cache: bool = True, unpad_params=None):
        out, next_cache = self.self_attention(input, attention_mask, attention_bias, pos_emb, cache,
                                              use_cache, unpad_params)
        out = _run_ff(self, self.ff, out)
        rest = None
        if isinstance(out, tuple):
            out, rest = out
        return out, residual, next_cache, rest


class FusedTransformerEncoderBlock(nn.Module):
    """Pre-norm block that carries the un-normalised residual stream separately so each
    residual add is fused into the following RMSNorm kernel:
        (h, res) -> norm(h + res) -> attention -> (a, h + res) -> norm(a + res') -> ff -> ...
    The final add happens in the model's `post_blocks`."""

    def __init__(self, self_attention, ff):
        super().__init__()
        self.self_attention = self_attention   # ResidualBlock-shaped: pre_norm + module
        self.ff = ff

    def forward(self, input, residual=None, attention_mask=None, attention_bias=None, pos_emb=None,
                cache=None, use_cache=True, unpad_params=None):
        sa, ff = self.self_attention, self.ff
        if residual is None:
            residual = input
            normed = sa.pre_norm(input)
        else:
            normed, residual = sa.pre_norm(input, residual)
        out, next_cache = sa.module(normed, attention_mask, attention_bias, pos_emb, cache, use_cache,
                                    unpad_params)
        normed, residual = ff.pre_norm(out, residual)
        out = _run_ff(self, ff.module, normed)
        rest = None
        if isinstance(out, tuple):
            out, rest = out
        return out, residual, next_cache, rest


class NGPTBlock(nn.Module):
    """Normalised-GPT update: x <- norm(x + scale * (norm(module(x)) - x))."""

    def __init__(self, module, post_norm=None, skip_norm=None, scale=None, dropout=0):
        super().__init__()
        self.module = module
        self.post_norm = post_norm
        self.skip_norm = skip_norm
        self.scale = scale
        self.dropout = nn.Dropout(dropout)

    def forward(self, input, *args, **kwargs):
        out = self.module(input, *args, **kwargs)
        rest = None
        if isinstance(out, tuple):
            out, *rest = out
        if self.post_norm is not None:
            out = self.post_norm(out)
        out = out - input
        if self.scale is not None:
            out = self.scale(out)
        out = input + self.dropout(out)
        if self.skip_norm is not None:
            out = self.skip_norm(out)
        if rest is not None:
            return (out, *rest)
        return out

    def tp_plan(self):
        plan = {}
        if self.post_norm is not None:
            plan["post_norm"] = "sequence"
        if self.skip_norm is not None:
            plan["skip_norm"] = "sequence"
        return plan
