"""Attention-mask programs (reference: transformers/flex_attention/*.py).

Each mask class keeps the reference's calling convention: called with its declared `inputs` it
returns a `mask_mod(b, h, q_idx, kv_idx) -> bool` (True = may attend). On top of that every
class carries a structured description (`MaskSpec`): whether it is causal, its window, and the
per-batch document offsets. `FlexAttentionProcessor` returns a `ResolvedMask` that the
attention dispatcher turns either into kernel arguments (causal flag, window, per-row document
offsets, which become per-token segment bounds on the device) or, for arbitrary programs and
score modifiers, into a dense boolean mask evaluated once per batch and cached according to the
update mode.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Callable, NamedTuple

import torch
from torch import nn


class FlexAttentionUpdateMode(Enum):
    NEVER = "never"
    BATCH = "batch"
    LAYER = "layer"


@dataclass
class MaskSpec:
    """What a mask program means, when it can be said without running it per element."""

    causal: bool = False
    window: int | None = None
    document_offsets: torch.Tensor | None = None     # [B, n_docs + 1] cumulative lengths
    opaque: bool = False                              # True: only the mask_mod describes it


class FlexAttentionInput(NamedTuple):
    score_mod: Callable | None
    block_mask: "ResolvedMask | None"


class ResolvedMask:
    """Outcome of a mask program for one batch."""

    def __init__(self, mask_mod, spec: MaskSpec, batch, n_heads, q_len, kv_len, score_mod=None):
        self.mask_mod, self.spec = mask_mod, spec
        self.batch, self.n_heads, self.q_len, self.kv_len = batch, n_heads, q_len, kv_len
        self.score_mod = score_mod
        self._dense = None

    def dense(self, device):
        """[B or 1, H or 1, Q, K] boolean, True = blocked (the convention of the eager attention)."""
        if self._dense is None or self._dense.device != torch.device(device):
            b = torch.arange(self.batch, device=device).view(-1, 1, 1, 1)
            h = torch.arange(self.n_heads or 1, device=device).view(1, -1, 1, 1)
            q = torch.arange(self.q_len, device=device).view(1, 1, -1, 1)
            k = torch.arange(self.kv_len, device=device).view(1, 1, 1, -1)
            allowed = self.mask_mod(b, h, q, k)
            self._dense = ~allowed.expand(self.batch, self.n_heads or 1, self.q_len, self.kv_len)
        return self._dense

    def to_attention_kwargs(self, q_len, kv_len, device):
        s = self.spec
        if not s.opaque and self.score_mod is None:
            # causal flag, window and per-row document offsets are arguments of the attention
            # kernel; only programs that cannot be described that way are evaluated densely
            out = {"causal": s.causal, "window": s.window}
            if s.document_offsets is not None:
                out["document_offsets"] = s.document_offsets
            return out
        return {"causal": False, "window": None, "mask": self.dense(device)}


class FlexAttentionProcessor(nn.Module):
    def __init__(self, score_mod=None, block_mask=None, n_heads: int | None = None, compile: bool = True):
        super().__init__()
        self.score_mod, self.block_mask = score_mod, block_mask
        self.n_heads = n_heads
        self.batch_shared = False
        if block_mask is not None:
            if getattr(block_mask, "head_shared", True):
                self.n_heads = None
            self.batch_shared = getattr(block_mask, "batch_shared", False)
        never = FlexAttentionUpdateMode.NEVER
        self.score_mod_update_mode = getattr(score_mod, "update_mode", never)
        self.block_mask_update_mode = getattr(block_mask, "update_mode", never)
        self.score_mod_inputs = getattr(score_mod, "inputs", ())
        self.block_mask_inputs = getattr(block_mask, "inputs", ())
        self.compile = compile          # accepted for compatibility; nothing is traced here
        self._cached = None
        self._cached_key = None

    def forward(self, batch, q_len, kv_len, device="cuda", **kwargs):
        key = (batch, q_len, kv_len)
        if self._cached is not None and self._cached_key == key and \
                self.block_mask_update_mode == FlexAttentionUpdateMode.NEVER and \
                self.score_mod_update_mode == FlexAttentionUpdateMode.NEVER:
            return self._cached
        kwargs.update(batch=batch, n_heads=self.n_heads, q_len=q_len, kv_len=kv_len, device=device)
        score_mod = None
        if self.score_mod is not None:
            score_mod = self.score_mod(**{k: kwargs[k] for k in self.score_mod_inputs})
        mask_mod, spec = None, MaskSpec()
        if self.block_mask is not None:
            args = {k: kwargs[k] for k in self.block_mask_inputs}
            mask_mod = self.block_mask(**args)
            spec = self.block_mask.spec(**args) if hasattr(self.block_mask, "spec") else MaskSpec(opaque=True)
        out = ResolvedMask(mask_mod, spec, 1 if self.batch_shared else batch, self.n_heads, q_len, kv_len,
                           score_mod)
        self._cached, self._cached_key = out, key
        return out


from .causal import CausalMask, causal_mask  # noqa: E402
from .sliding_window import SlidingWindowCausalMask  # noqa: E402
from .batch_document_mask import BatchDocumentMask, batch_length_to_offsets  # noqa: E402
from .bidirectional import BidirectionalMask  # noqa: E402
from .mask import ComposeMask  # noqa: E402

__all__ = ["FlexAttentionUpdateMode", "FlexAttentionInput", "FlexAttentionProcessor", "MaskSpec", "ResolvedMask",
           "CausalMask", "causal_mask", "SlidingWindowCausalMask", "BatchDocumentMask", "batch_length_to_offsets",
           "BidirectionalMask", "ComposeMask"]
