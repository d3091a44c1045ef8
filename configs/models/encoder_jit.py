"""Encoder-JiT builder: conditional JiT blocks on top of a (pretrained) vision encoder's patch
embedding and blocks (reference: configs/models/encoder_jit.py). `encoder_jit(...)` returns a
partial that the trainer calls with the loaded encoder: `EncoderJiT(encoder, ...)`."""

from copy import deepcopy
from functools import partial

from halite_b200.conf import call, config_fn
from halite_b200.models.models.jit import (EncoderJiT, InContextEmbedding, JiTHead, JiTModulator, LabelEmbedding,
                                           TimeEmbedding, VisionRoPE, apply_vision_rope)
from halite_b200.nn.normalization import RMSNorm

from .jit import build_block, use_flash_attention  # noqa: F401  (re-exported for experiment files)


@config_fn
def encoder_jit(image_size, patch_size, n_labels, dim, patch_dim, n_heads, head_dim, n_layers, intermediate_size,
                in_context_len, in_context_start=0, n_key_value_heads=None, rms_norm_epsilon=1e-6,
                attention_processor="auto", attention_bias=True, ffn_bias=True, ffn_activation="swiglu",
                qk_norm=False, cond_start_id=0):
    grid = image_size // patch_size
    rope_dim = head_dim // 2
    blocks = []
    for i in range(n_layers):
        qn = RMSNorm(head_dim, eps=rms_norm_epsilon) if qk_norm else None
        blocks.append(call[build_block](i, dim, n_heads, head_dim, intermediate_size, n_key_value_heads,
                                        rms_norm_epsilon, partial(apply_vision_rope), attention_processor,
                                        attention_bias, ffn_bias, ffn_activation, q_norm=qn, k_norm=deepcopy(qn)))
    return partial(
        EncoderJiT,
        time_embedding=TimeEmbedding(dim), label_embedding=LabelEmbedding(n_labels, dim),
        in_context_embed=InContextEmbedding(dim, in_context_len),
        in_context_rope=VisionRoPE(rope_dim, grid, in_context_len), blocks=blocks,
        head=JiTHead(RMSNorm(dim, eps=rms_norm_epsilon), JiTModulator(dim, 2), dim, 3, patch_size),
        cond_start_id=cond_start_id)
