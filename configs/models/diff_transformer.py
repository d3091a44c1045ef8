"""Differential Transformer: attention = softmax(Q1 K1^T) - lambda * softmax(Q2 K2^T), lambda
re-parameterised per layer with a depth-dependent initial value
(reference: configs/models/diff_transformer.py)."""

import math
from copy import deepcopy
from functools import partial

from torch import nn

from halite_b200.conf import call, config_fn, field
from halite_b200.models.attention import DiffAttention, SelfAttention, SelfAttentionQKV
from halite_b200.models.block import ResidualBlock, TransformerEncoderBlock
from halite_b200.models.embedding import TextEmbedding
from halite_b200.models.feedforward import (FeedForward, GatedFeedForward, SequenceParallelWrapper,
                                            VocabParallelLinear)
from halite_b200.models.position import RotaryEmbedding, apply_rotary_emb
from halite_b200.models.transformer import TransformerDecoder
from halite_b200.nn.activation import SwiGLU
from halite_b200.nn.normalization import RMSNorm


@config_fn
def build_block(layer_id, dim, n_heads, n_layers, intermediate_size, softcap=0.0, rms_norm_epsilon=1e-6,
                post_norm=False, attention_processor="native", qkv_split=False, gated_ff_split=False):
    init = partial(nn.init.kaiming_normal_, nonlinearity="linear")
    attention = DiffAttention(
        n_heads, dim // n_heads // 2, lambda_init=0.8 - 0.6 * call[math.exp](-0.3 * layer_id),
        sub_norm=RMSNorm(dim // n_heads * 2, eps=1e-5, elementwise_affine=False), attn_drop=0,
        apply_pos_emb_fn=partial(apply_rotary_emb), processor=attention_processor, softcap=softcap, is_causal=True)
    norm = RMSNorm(dim, eps=rms_norm_epsilon)
    norm_post = RMSNorm(dim, eps=rms_norm_epsilon, weight_init=partial(nn.init.constant_, val=n_layers ** -0.5))
    if qkv_split:
        self_attention = SelfAttentionQKV(
            q=nn.Linear(dim, dim, bias=False), k=nn.Linear(dim, dim, bias=False), v=nn.Linear(dim, dim, bias=False),
            attention=attention, out=nn.Linear(dim, dim, bias=False), q_init=init, k_init=init, v_init=init,
            out_init=init)
    else:
        self_attention = SelfAttention(qkv=nn.Linear(dim, dim * 3, bias=False), attention=attention,
                                       out=nn.Linear(dim, dim, bias=False), qkv_split="llama", qkv_init=init,
                                       out_init=init)
    if gated_ff_split:
        ff = GatedFeedForward(nn.Linear(dim, intermediate_size, bias=False),
                              nn.Linear(dim, intermediate_size, bias=False), nn.SiLU(),
                              nn.Linear(intermediate_size, dim, bias=False), linear_proj_init=init,
                              linear_gate_init=init, linear_out_init=init)
    else:
        ff = FeedForward(nn.Linear(dim, intermediate_size * 2, bias=False), SwiGLU(),
                         nn.Linear(intermediate_size, dim, bias=False), linear1_init=init, linear2_init=init)
    return TransformerEncoderBlock(
        ResidualBlock(deepcopy(norm), self_attention, post_norm=deepcopy(norm_post) if post_norm else None),
        ResidualBlock(deepcopy(norm), ff, post_norm=deepcopy(norm_post) if post_norm else None))


@config_fn
def diff_transformer(vocab_size, dim, n_heads, n_layers, intermediate_size, max_position_embeddings, softcap=0.0,
                     rms_norm_epsilon=1e-6, post_norm=False, attention_processor="native", qkv_split=False,
                     gated_ff_split=False):
    init = partial(nn.init.kaiming_normal_, nonlinearity="linear")
    blocks = [call[build_block](i, dim, n_heads, n_layers, intermediate_size, softcap, rms_norm_epsilon, post_norm,
                                attention_processor, qkv_split, gated_ff_split) for i in range(n_layers)]
    return TransformerDecoder(
        embedding=TextEmbedding(nn.Embedding(vocab_size, dim), 0, embed_init=init, multiplier=dim ** 0.5),
        pos_embed=RotaryEmbedding(dim // n_heads // 2, max_position_embeddings), blocks=blocks,
        post_blocks=SequenceParallelWrapper(RMSNorm(dim, eps=rms_norm_epsilon)),
        head=VocabParallelLinear(nn.Linear(dim, vocab_size, bias=False), linear_init=init),
        tie_embeds=False, use_position_ids=True, attention_processor=attention_processor)


conf = field(model=call[diff_transformer](32000, 96, 4, 3, call[int](96 * 3.5), 2048, 1e-6))
