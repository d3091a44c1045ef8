"""Packed-document masking: several documents stacked in one row attend only within
themselves, with an inner mask applied to document-local positions
(reference: transformers/flex_attention/batch_document_mask.py)."""

import torch

from . import FlexAttentionUpdateMode, MaskSpec


def batch_length_to_offsets(lengths, device="cpu"):
    """[[len, ...] per row] -> [B, max_docs + 1] cumulative offsets, padded by repeating the end."""
    width = max(len(row) for row in lengths) + 1
    out = torch.zeros(len(lengths), width, dtype=torch.int32, device=device)
    for i, row in enumerate(lengths):
        c = torch.tensor([0] + list(row), dtype=torch.int32, device=device).cumsum(0)
        out[i, :len(c)] = c
        out[i, len(c):] = c[-1]
    return out


def _doc_ids(offsets, length=None):
    """offsets [B, n+1] -> document id of every position [B, L]."""
    length = int(offsets[:, -1].max()) if length is None else length
    pos = torch.arange(length, device=offsets.device)
    # number of document starts (excluding the first) at or before each position
    return (pos[None, :, None] >= offsets[:, None, 1:]).sum(-1)


class BatchDocumentMask:
    inputs: tuple = ("document_offsets",)
    update_mode = FlexAttentionUpdateMode.BATCH
    head_shared = True
    batch_shared = False

    def __init__(self, mask_mod):
        if isinstance(mask_mod, type):
            mask_mod = mask_mod()
        self.inner = mask_mod
        self.mask_mod_fn = mask_mod()

    def __call__(self, document_offsets):
        doc = _doc_ids(document_offsets)
        last = doc.shape[1] - 1
        inner = self.mask_mod_fn
        n_off = document_offsets.shape[1]

        def doc_mask_mod(b, h, q_idx, kv_idx):
            qd = doc[b, q_idx.clamp(max=last)]
            kd = doc[b, kv_idx.clamp(max=last)]
            q_local = q_idx - document_offsets[b, qd.clamp(max=n_off - 1)]
            kv_local = kv_idx - document_offsets[b, kd.clamp(max=n_off - 1)]
            return (qd == kd) & inner(b, h, q_local, kv_local)

        return doc_mask_mod

    def spec(self, document_offsets):
        s = self.inner.spec() if hasattr(self.inner, "spec") else MaskSpec(opaque=True)
        return MaskSpec(causal=s.causal, window=s.window, document_offsets=document_offsets, opaque=s.opaque)
