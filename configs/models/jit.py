"""JiT pixel-space diffusion transformer builder (reference: configs/models/jit.py)."""

from copy import deepcopy
from functools import partial

from torch import nn

from halite_b200.conf import call, config_fn, select
from halite_b200.models.attention import Attention, SelfAttention
from halite_b200.models.embedding import PatchEmbedding
from halite_b200.models.feedforward import FeedForward
from halite_b200.models.models.jit import (BottleneckEmbedding, InContextEmbedding, JiT, JiTBlock, JiTHead,
                                           JiTModulator, LabelEmbedding, SinusoidalEmbedding, TimeEmbedding,
                                           VisionRoPE, apply_vision_rope)
from halite_b200.nn.activation import GEGLU, SwiGLU
from halite_b200.nn.normalization import RMSNorm

_ACTIVATIONS = {"swiglu": (SwiGLU(), True), "gelu_tanh": (nn.GELU(approximate="tanh"), False),
                "geglu_tanh": (GEGLU(approximate="tanh"), True)}


@config_fn
def get_activation(activation):
    return _ACTIVATIONS.get(activation)


@config_fn
def build_block(layer_id, dim, n_heads, head_dim, intermediate_size, n_key_value_heads=None, rms_norm_epsilon=1e-6,
                pos_embed_apply_fn=None, attention_processor="auto", attention_bias=False, ffn_bias=False,
                ffn_activation="swiglu", q_norm=None, k_norm=None):
    xavier = partial(nn.init.xavier_uniform_)
    kv = n_key_value_heads if n_key_value_heads is not None else n_heads
    attention = Attention(n_heads, head_dim, n_key_value_heads=n_key_value_heads, attn_drop=0,
                          apply_pos_emb_fn=pos_embed_apply_fn, processor=attention_processor, is_causal=False,
                          q_norm=deepcopy(q_norm), k_norm=deepcopy(k_norm))
    self_attention = SelfAttention(qkv=nn.Linear(dim, head_dim * (n_heads + 2 * kv), bias=attention_bias),
                                   attention=attention, out=nn.Linear(head_dim * n_heads, dim, bias=attention_bias),
                                   qkv_split="llama", qkv_init=xavier, out_init=xavier)
    act, gated = call[get_activation](ffn_activation)
    ff = FeedForward(nn.Linear(dim, intermediate_size * (2 if gated else 1), bias=ffn_bias), deepcopy(act),
                     nn.Linear(intermediate_size, dim, bias=ffn_bias), linear1_init=xavier, linear2_init=xavier)
    norm = RMSNorm(dim, eps=rms_norm_epsilon)
    return JiTBlock(JiTModulator(dim, 6), deepcopy(norm), self_attention, deepcopy(norm), ff)


@config_fn
def jit(image_size, patch_size, n_labels, dim, patch_dim, n_heads, head_dim, n_layers, intermediate_size,
        in_context_len, in_context_start=0, n_key_value_heads=None, rms_norm_epsilon=1e-6,
        attention_processor="auto", attention_bias=True, ffn_bias=True, ffn_activation="swiglu", qk_norm=False):
    xavier = partial(nn.init.xavier_uniform_)
    grid = image_size // patch_size
    rope_dim = head_dim // 2
    blocks = []
    for i in range(n_layers):
        qn = RMSNorm(head_dim, eps=rms_norm_epsilon) if qk_norm else None
        blocks.append(call[build_block](i, dim, n_heads, head_dim, intermediate_size, n_key_value_heads,
                                        rms_norm_epsilon, partial(apply_vision_rope), attention_processor,
                                        attention_bias, ffn_bias, ffn_activation, q_norm=qn, k_norm=deepcopy(qn)))
    return JiT(
        embedding=PatchEmbedding(3, patch_dim, patch_size, use_bias=False, patch_embedding_init=xavier),
        time_embedding=TimeEmbedding(dim), label_embedding=LabelEmbedding(n_labels, dim),
        post_embed=BottleneckEmbedding(patch_dim, dim, linear_init=xavier),
        pos_embed=SinusoidalEmbedding(dim, grid, grid * grid), pos_rope=VisionRoPE(rope_dim, grid),
        in_context_embed=InContextEmbedding(dim, in_context_len),
        in_context_rope=VisionRoPE(rope_dim, grid, in_context_len), in_context_start=in_context_start,
        blocks=blocks, head=JiTHead(RMSNorm(dim, eps=rms_norm_epsilon), JiTModulator(dim, 2), dim, 3, patch_size))


@config_fn
def use_flash_attention(model_conf):
    return select(model_conf).instance(Attention).update_dict(dict(processor="flash_attn"))
