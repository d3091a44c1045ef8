"""Plain causal mask (reference: transformers/flex_attention/causal.py)."""

from . import FlexAttentionUpdateMode, MaskSpec


def causal_mask(b, h, q_idx, kv_idx):
    return q_idx >= kv_idx


class CausalMask:
    inputs: tuple = ()
    update_mode = FlexAttentionUpdateMode.NEVER
    head_shared = True
    batch_shared = True

    def __call__(self):
        return causal_mask

    def spec(self):
        return MaskSpec(causal=True)
