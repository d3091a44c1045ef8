"""Inference block (reference: infer/block.py): same sub-modules as the training block, flat
activations, a ForwardBatch instead of masks and caches."""

from __future__ import annotations

from torch import nn


class InferTransformerEncoderBlock(nn.Module):
    def __init__(self, self_attention, ff):
        super().__init__()
        self.self_attention = self_attention
        self.ff = ff

    def forward(self, input, forward_batch, pos_emb=None):
        out = self.self_attention(input, forward_batch, pos_emb)
        out = self.ff(out)
        if isinstance(out, tuple):
            out = out[0]
        return out
