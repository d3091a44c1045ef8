"""Causal mask limited to the last `window_size` keys (reference: transformers/flex_attention/sliding_window.py)."""

from . import FlexAttentionUpdateMode, MaskSpec


class SlidingWindowCausalMask:
    inputs: tuple = ()
    update_mode = FlexAttentionUpdateMode.NEVER
    head_shared = True
    batch_shared = True

    def __init__(self, window_size: int):
        self.window_size = window_size

    def __call__(self):
        w = self.window_size

        def sliding_window_causal_mask(b, h, q_idx, kv_idx):
            return (q_idx >= kv_idx) & (q_idx - kv_idx <= w)

        return sliding_window_causal_mask

    def spec(self):
        return MaskSpec(causal=True, window=self.window_size)
