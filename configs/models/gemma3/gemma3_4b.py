"""Gemma-3-4B multimodal: SigLIP2-so400m vision tower -> 256 soft tokens per image -> a 34-layer
decoder that alternates five sliding-window (1024) layers with one global layer, `(1+w)` RMSNorm
before and after every sub-layer, q/k norm, GeGLU, tied embeddings; image tokens attend to each
other bidirectionally."""

from functools import partial

from torch import nn

from halite_b200.conf import call, field, function
from halite_b200.models.container import MultiModule
from halite_b200.models.embedding import MultiModalEmbedding
from halite_b200.models.flex_attention import (BidirectionalMask, CausalMask, FlexAttentionProcessor,
                                                SlidingWindowCausalMask)
from halite_b200.models.position import LinearRoPE, RotaryEmbedding, apply_rotary_emb
from halite_b200.models.variants.gemma3 import MultiModalProjector, RMSNorm, TextEmbedding
from halite_b200.parallel.parallelize import parallelize

from ..siglip2.siglip_vision import vision_config
from ..transformer import transformer
from .checkpoint import to_halite_postprocess, weight_maps

conf = field()

image_size, patch_size = 896, 14
siglip_dim = 1152
siglip = call[transformer](**vision_config(siglip_dim, 16, 27, 4304, image_size, patch_size))

n_vocab, dim, n_layers, n_heads, head_dim = 262208, 2560, 34, 8, 256
context_len = 131072
image_token_id = 262144
sliding_window_ratio = 6
layer_types = ["local_attn" if (i + 1) % sliding_window_ratio != 0 else "global_attn" for i in range(n_layers)]

decoder_config = field(
    vocab_size=n_vocab, dim=dim, n_heads=n_heads, head_dim=head_dim, n_layers=n_layers, context_len=context_len,
    intermediate_size=10240, norm=RMSNorm(dim, eps=1e-6), attention_bias=False, attention_processor="flex",
    n_key_value_heads=4,
    flex_attention_processor=MultiModule(
        local_attn=FlexAttentionProcessor(block_mask=BidirectionalMask(SlidingWindowCausalMask(1024))),
        global_attn=FlexAttentionProcessor(block_mask=BidirectionalMask(CausalMask()))),
    is_causal=False, ffn_bias=False, ffn_activation="geglu_tanh",
    pos_embed=MultiModule(
        local_attn=RotaryEmbedding(head_dim, context_len, base=10000.0, use_rotate_half=True),
        global_attn=LinearRoPE(head_dim, context_len, base=1000000.0, scaling=8.0, use_rotate_half=True)),
    pos_embed_apply_fn=partial(apply_rotary_emb),
    post_norm=True,
    embedding=MultiModalEmbedding(
        text_embedding=TextEmbedding(nn.Embedding(n_vocab, dim), multiplier=dim ** 0.5),
        image_embedding=MultiModalProjector(siglip, siglip_dim, dim, 1e-6, image_size, patch_size, 256),
        image_mask_token_id=image_token_id),
    qkv_split=True, gated_ff_split=True,
    q_norm=RMSNorm(head_dim, eps=1e-6), k_norm=RMSNorm(head_dim, eps=1e-6),
    tie_embeds=True, layer_types=layer_types,
)

conf.model = call[transformer](**decoder_config)
conf.model_conf = field(vocab_size=n_vocab, dim=dim, n_heads=n_heads, head_dim=head_dim, n_layers=n_layers,
                        n_key_value_heads=4, intermediate_size=10240, context_len=context_len, qkv_split=True,
                        gated_ff_split=True, tie_embeds=True, dtype="bfloat16")
conf.parallelize = partial(parallelize, param_dtype="bfloat16", reduce_dtype="float32")
conf.policy = field(weight_maps=weight_maps, to_halite_postprocess=function(to_halite_postprocess))
