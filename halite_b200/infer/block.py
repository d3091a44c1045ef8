"""Inference block (reference: infer/block.py): same sub-modules as the training block, flat
activations, a ForwardBatch instead of masks and caches.

When both halves are plain pre-norm residual blocks with RMSNorm, the block carries the
un-normalised residual stream next to its output, so every residual add runs inside the
following RMSNorm kernel (two launches fewer per layer and decode step); the decoder's final norm
does the last add."""

from __future__ import annotations

from torch import nn

from halite_b200.models.block import ResidualBlock
from halite_b200.nn.normalization import RMSNorm


def _plain_prenorm(block):
    return (isinstance(block, ResidualBlock) and isinstance(block.pre_norm, RMSNorm) and block.post_norm is None
            and block.pre_norm.weight is not None and (not block.training or block.dropout.p == 0))


class InferTransformerEncoderBlock(nn.Module):
    def __init__(self, self_attention, ff):
        super().__init__()
        self.self_attention = self_attention
        self.ff = ff

    def fuses_residual(self):
        return _plain_prenorm(self.self_attention) and _plain_prenorm(self.ff)

    def forward(self, input, forward_batch, pos_emb=None):
        out = self.self_attention(input, forward_batch, pos_emb)
        out = self.ff(out)
        if isinstance(out, tuple):
            out = out[0]
        return out

    def forward_fused(self, input, residual, forward_batch, pos_emb=None):
        """(h, res) -> (ff output, h + res + attention output): the adds happen in the norms."""
        sa, ff = self.self_attention, self.ff
        if residual is None:
            residual = input
            normed = sa.pre_norm(input)
        else:
            normed, residual = sa.pre_norm(input, residual)
        out = sa.module(normed, forward_batch, pos_emb)
        normed, residual = ff.pre_norm(out, residual)
        out = ff.module(normed)
        if isinstance(out, tuple):
            out = out[0]
        return out, residual
