"""Decoder whose feed-forward is a top-k mixture of SwiGLU experts
(reference: configs/models/moe_transformer.py:25-147)."""

from copy import deepcopy
from functools import partial

from torch import nn

from halite_b200.conf import config_fn
from halite_b200.models.attention import Attention, SelfAttention, SelfAttentionQKV
from halite_b200.models.block import ResidualBlock, TransformerEncoderBlock
from halite_b200.models.embedding import TextEmbedding
from halite_b200.models.feedforward import SequenceParallelWrapper, VocabParallelLinear
from halite_b200.models.moe import ExpertLinear, FeedForward, MoE, TopKRouter
from halite_b200.models.position import RotaryEmbedding, apply_rotary_emb
from halite_b200.models.transformer import TransformerDecoder
from halite_b200.nn.activation import SwiGLU
from halite_b200.nn.init import kaiming_normal_
from halite_b200.nn.normalization import RMSNorm


@config_fn
def moe_transformer(vocab_size, dim, n_heads, n_layers, n_experts, expert_top_k, z_loss, load_balance_loss,
                    intermediate_size, max_position_embeddings, softcap=0.0, rms_norm_epsilon=1e-6, post_norm=False,
                    attention_processor="native", qkv_split=False, capacity_factor=None, token_dispatcher=None):
    init = partial(kaiming_normal_, nonlinearity="linear", truncate=3)
    head_dim = dim // n_heads
    attention = Attention(n_heads, head_dim, attn_drop=0, apply_pos_emb_fn=partial(apply_rotary_emb),
                          processor=attention_processor, softcap=softcap, is_causal=True)
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
    ff = MoE(
        TopKRouter(dim, n_experts, expert_top_k, gate_init=init, z_loss=z_loss, load_balance_loss=load_balance_loss,
                   capacity_factor=capacity_factor, pre_softmax=True, deterministic=True),
        token_dispatcher,
        FeedForward(ExpertLinear(n_experts, dim, intermediate_size * 2), SwiGLU(),
                    ExpertLinear(n_experts, intermediate_size, dim), top_k=expert_top_k, linear1_init=init,
                    linear2_init=init))
    block = TransformerEncoderBlock(
        ResidualBlock(deepcopy(norm), self_attention, post_norm=deepcopy(norm_post) if post_norm else None),
        ResidualBlock(deepcopy(norm), ff, post_norm=deepcopy(norm_post) if post_norm else None))
    blocks = [deepcopy(block) for _ in range(n_layers)]
    return TransformerDecoder(
        embedding=TextEmbedding(nn.Embedding(vocab_size, dim), 0, embed_init=init, multiplier=dim ** 0.5),
        pos_embed=RotaryEmbedding(head_dim, max_position_embeddings), blocks=blocks,
        post_blocks=SequenceParallelWrapper(RMSNorm(dim, eps=rms_norm_epsilon)),
        head=VocabParallelLinear(nn.Linear(dim, vocab_size, bias=False), linear_init=init),
        tie_embeds=False, use_position_ids=True, attention_processor=attention_processor)
