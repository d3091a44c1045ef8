"""Dense decoder family used for scaling-law sweeps: RMSNorm, RoPE, SwiGLU, optional depth-scaled
post-norm, embedding scaled by sqrt(dim) (reference: configs/models/scaling/base.py:26-157)."""

from copy import deepcopy
from functools import partial

from torch import nn

from halite_b200.conf import call, config_fn, field
from halite_b200.models.attention import Attention, SelfAttention, SelfAttentionQKV
from halite_b200.models.block import ResidualBlock, TransformerEncoderBlock
from halite_b200.models.config import TransformerConfig
from halite_b200.models.embedding import TextEmbedding
from halite_b200.models.feedforward import (FeedForward, GatedFeedForward, SequenceParallelWrapper,
                                            VocabParallelLinear)
from halite_b200.models.position import RotaryEmbedding, apply_rotary_emb
from halite_b200.models.transformer import TransformerDecoder
from halite_b200.nn.activation import SwiGLU
from halite_b200.nn.normalization import RMSNorm


@config_fn
def transformer(vocab_size, dim, n_heads, head_dim, n_layers, intermediate_size, max_position_embeddings,
                softcap=0.0, rms_norm_epsilon=1e-6, post_norm=False, attention_processor="native", qkv_split=False,
                gated_ff_split=False):
    init = partial(nn.init.kaiming_normal_, nonlinearity="linear")
    attention = Attention(n_heads, head_dim, attn_drop=0, apply_pos_emb_fn=partial(apply_rotary_emb),
                          processor=attention_processor, softcap=softcap, is_causal=True)
    norm = RMSNorm(dim, eps=rms_norm_epsilon)
    norm_post = RMSNorm(dim, eps=rms_norm_epsilon, weight_init=partial(nn.init.constant_, val=n_layers ** -0.5))
    inner = n_heads * head_dim
    if qkv_split:
        self_attention = SelfAttentionQKV(
            q=nn.Linear(dim, inner, bias=False), k=nn.Linear(dim, inner, bias=False),
            v=nn.Linear(dim, inner, bias=False), attention=attention, out=nn.Linear(inner, dim, bias=False),
            q_init=init, k_init=init, v_init=init, out_init=init)
    else:
        self_attention = SelfAttention(qkv=nn.Linear(dim, inner * 3, bias=False), attention=attention,
                                       out=nn.Linear(inner, dim, bias=False), qkv_split="llama", qkv_init=init,
                                       out_init=init)
    if gated_ff_split:
        ff = GatedFeedForward(nn.Linear(dim, intermediate_size, bias=False),
                              nn.Linear(dim, intermediate_size, bias=False), nn.SiLU(),
                              nn.Linear(intermediate_size, dim, bias=False), linear_proj_init=init,
                              linear_gate_init=init, linear_out_init=init)
    else:
        ff = FeedForward(nn.Linear(dim, intermediate_size * 2, bias=False), SwiGLU(),
                         nn.Linear(intermediate_size, dim, bias=False), linear1_init=init, linear2_init=init)
    block = TransformerEncoderBlock(
        ResidualBlock(deepcopy(norm), self_attention, post_norm=deepcopy(norm_post) if post_norm else None),
        ResidualBlock(deepcopy(norm), ff, post_norm=deepcopy(norm_post) if post_norm else None))
    return TransformerDecoder(
        embedding=TextEmbedding(nn.Embedding(vocab_size, dim), 0, embed_init=init, multiplier=dim ** 0.5),
        pos_embed=RotaryEmbedding(head_dim, max_position_embeddings),
        blocks=[deepcopy(block) for _ in range(n_layers)],
        post_blocks=SequenceParallelWrapper(RMSNorm(dim, eps=rms_norm_epsilon)),
        head=VocabParallelLinear(nn.Linear(dim, vocab_size, bias=False), linear_init=init),
        tie_embeds=False, use_position_ids=True, attention_processor=attention_processor,
        config=TransformerConfig(dim=dim, n_heads=n_heads, head_dim=head_dim, n_layers=n_layers,
                                 vocab_size=vocab_size, intermediate_size=intermediate_size,
                                 context_len=max_position_embeddings))


conf = field(model=call[transformer](32000, 96, 4, 24, 3, call[int](96 * 3.5), 2048, 1e-6))
