"""Last-token gather + head projection to fp32 logits (reference: infer/postprocessor.py:9-57)."""

from __future__ import annotations

import torch
from torch import nn

from halite_b200 import ops


class LogitsProcessor(nn.Module):
    def forward(self, hidden, head_weight, forward_batch, scale=None):
        if not forward_batch.mode.is_decode():
            hidden = hidden.index_select(0, forward_batch.sample_indices)
        logits = ops.matmul_nt(hidden, head_weight, out_dtype=torch.float32)
        if scale is not None:
            logits = logits * scale
        return logits
