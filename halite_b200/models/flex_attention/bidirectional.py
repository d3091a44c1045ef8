"""Positions sharing a positive `bidirection_id` see each other in both directions (image
spans inside causal text); everything else follows the inner mask
(reference: transformers/flex_attention/bidirectional.py)."""

from . import FlexAttentionUpdateMode, MaskSpec


class BidirectionalMask:
    inputs: tuple = ("bidirection_ids",)
    update_mode = FlexAttentionUpdateMode.BATCH
    head_shared = True
    batch_shared = False

    def __init__(self, mask_mod):
        if isinstance(mask_mod, type):
            mask_mod = mask_mod()
        self.mask_mod_fn = mask_mod()

    def __call__(self, bidirection_ids):
        inner = self.mask_mod_fn
        if bidirection_ids is None:          # text-only batch: just the inner mask
            return inner
        last = bidirection_ids.shape[1] - 1

        def bidirectional_mask_mod(b, h, q_idx, kv_idx):
            qi = bidirection_ids[b, q_idx.clamp(max=last)]
            ki = bidirection_ids[b, kv_idx.clamp(max=last)]
            return ((qi > 0) & (qi == ki)) | inner(b, h, q_idx, kv_idx)

        return bidirectional_mask_mod

    def spec(self, bidirection_ids):
        return MaskSpec(opaque=True)
