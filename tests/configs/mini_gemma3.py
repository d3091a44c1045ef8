"""Miniature Gemma-3-style multimodal decoder for CPU tests (same structure as
configs/models/gemma3/gemma3_4b.py at toy sizes)."""

import os
from functools import partial

from torch import nn

from halite_b200.conf import call, field
from halite_b200.conf.loader import load_module
from halite_b200.models.container import MultiModule
from halite_b200.models.embedding import MultiModalEmbedding, PatchEmbedding
from halite_b200.models.flex_attention import (BidirectionalMask, CausalMask, FlexAttentionProcessor,
                                                SlidingWindowCausalMask)
from halite_b200.models.position import LearnedPositionEmbedding, LinearRoPE, RotaryEmbedding, apply_rotary_emb
from halite_b200.models.variants.gemma3 import MultiModalProjector, RMSNorm, TextEmbedding

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
_zoo = load_module(os.path.join(_ROOT, "configs/models/transformer.py"))
init = partial(nn.init.normal_, std=0.05)

vis = call[_zoo.transformer](
    vocab_size=0, dim=32, n_heads=2, head_dim=16, n_layers=1, context_len=16, intermediate_size=64,
    norm=nn.LayerNorm(32, eps=1e-6), pos_embed=None, attention_bias=True, is_causal=False, ffn_bias=True,
    ffn_activation="gelu_tanh",
    embedding=PatchEmbedding(3, 32, 4, LearnedPositionEmbedding(32, 16), use_bias=True, use_conv=True),
    qkv_split=True, use_head=False, init=init)

conf = field()
conf.model = call[_zoo.transformer](
    vocab_size=100, dim=48, n_heads=4, head_dim=16, n_layers=3, context_len=64, intermediate_size=96,
    norm=RMSNorm(48), attention_processor="flex", n_key_value_heads=2,
    flex_attention_processor=MultiModule(
        local_attn=FlexAttentionProcessor(block_mask=BidirectionalMask(SlidingWindowCausalMask(4))),
        global_attn=FlexAttentionProcessor(block_mask=BidirectionalMask(CausalMask()))),
    is_causal=False, ffn_activation="geglu_tanh",
    pos_embed=MultiModule(local_attn=RotaryEmbedding(16, 64, base=10000.0, use_rotate_half=True),
                          global_attn=LinearRoPE(16, 64, base=1000000.0, scaling=8.0, use_rotate_half=True)),
    pos_embed_apply_fn=partial(apply_rotary_emb), post_norm=True,
    embedding=MultiModalEmbedding(
        text_embedding=TextEmbedding(nn.Embedding(100, 48), multiplier=48 ** 0.5),
        image_embedding=MultiModalProjector(vis, 32, 48, 1e-6, 16, 4, 4), image_mask_token_id=99),
    qkv_split=True, gated_ff_split=True, q_norm=RMSNorm(16), k_norm=RMSNorm(16), tie_embeds=True,
    layer_types=["local_attn", "global_attn", "local_attn"], init=init)
