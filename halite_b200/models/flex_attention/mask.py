"""Intersection of several mask programs (reference: transformers/flex_attention/mask.py)."""

from . import FlexAttentionUpdateMode, MaskSpec


class ComposeMask:
    head_shared = True

    def __init__(self, *masks):
        self.masks = masks
        self.mask_inputs = [m.inputs for m in masks]
        self.inputs = tuple(sorted({name for m in masks for name in m.inputs}))
        modes = [m.update_mode for m in masks]
        self.update_mode = FlexAttentionUpdateMode.LAYER if FlexAttentionUpdateMode.LAYER in modes else \
            FlexAttentionUpdateMode.BATCH if FlexAttentionUpdateMode.BATCH in modes else FlexAttentionUpdateMode.NEVER
        self.batch_shared = all(getattr(m, "batch_shared", False) for m in masks)

    def __call__(self, **kwargs):
        mods = [m(**{k: kwargs[k] for k in names}) for m, names in zip(self.masks, self.mask_inputs)]

        def mask_mod(b, h, q_idx, kv_idx):
            out = mods[0](b, h, q_idx, kv_idx)
            for m in mods[1:]:
                out = out & m(b, h, q_idx, kv_idx)
            return out

        return mask_mod

    def spec(self, **kwargs):
        return MaskSpec(opaque=True)
