"""H-Net assembly: `hnet(arch, dims, ...)` builds the recursive encoder / main / decoder stages
(keyword surface of the reference's configs/models/hnet.py:330-392).

`arch` is nested: an innermost stage is `[layers]`; an outer stage is
`[encoder_layers, inner_arch_or_layers, decoder_layers]`, where each `*_layers` is a tuple of
`{"mixer": "mamba2" | "attention", "n_layer": n, "use_ffn": bool}` groups.
"""

from copy import deepcopy
from functools import partial

from halite_b200.conf import call, config_fn
from torch import nn

from halite_b200.nn.activation import GEGLU, SwiGLU
from halite_b200.nn.init import kaiming_linear_
from halite_b200.nn.normalization import RMSNorm
from halite_b200.models.attention import Attention, SelfAttention, SelfAttentionQKV
from halite_b200.models.block import ResidualBlock, TransformerEncoderBlock
from halite_b200.models.embedding import TextEmbedding
from halite_b200.models.feedforward import FeedForward, GatedFeedForward, VocabParallelLinear
from halite_b200.models.position import RotaryEmbedding, apply_rotary_emb
from halite_b200.models.models.hnet import HNet, HNetBlock, HNetDecoder, Mamba2Block
from halite_b200.models.models.mamba2 import Mamba2

ACTIVATIONS = {
    "swiglu": (SwiGLU(), nn.SiLU()),
    "gelu_tanh": (nn.GELU(approximate="tanh"), None),
    "geglu_tanh": (GEGLU(approximate="tanh"), nn.GELU(approximate="tanh")),
}


@config_fn
def get_activation(activation):
    return ACTIVATIONS.get(activation)


@config_fn
def get_value(map, key, default=None):
    return map.get(key, default)


@config_fn
def get_stage_kwargs(map_or_list, stage_idx):
    return map_or_list if isinstance(map_or_list, dict) else map_or_list[stage_idx]


@config_fn
def is_layer_group(item):
    """True for a tuple/list of layer-group dicts, False for a nested stage description."""
    return len(item) > 0 and all(isinstance(g, dict) for g in item)


@config_fn
def build_layer(layer_id, dim, intermediate_size, n_res_blocks, seq_mixer="attention", attn_kwargs=None,
                mamba2_kwargs=None, use_ffn=True, norm=None, rms_norm_epsilon=1e-6, post_norm=False,
                pos_embed_apply_fn=None, attn_bias=False, qkv_split=False, ffn_bias=False,
                ffn_activation="swiglu", gated_ff_split=False, fast_norm=False, q_norm=None, k_norm=None,
                layer_type=None):
    attn_kwargs = attn_kwargs or {}
    mamba2_kwargs = mamba2_kwargs or {}
    out_scale = 1 / (n_res_blocks ** 0.5)

    if seq_mixer == "mamba2":
        mixer = Mamba2Block(Mamba2(d_model=dim, **mamba2_kwargs), in_proj_init=partial(kaiming_linear_),
                            out_proj_init=partial(kaiming_linear_, scale=out_scale))
    else:
        n_heads, head_dim = attn_kwargs["n_heads"], attn_kwargs["head_dim"]
        kv_heads = attn_kwargs.get("n_key_value_heads") or n_heads
        core = Attention(**attn_kwargs, apply_pos_emb_fn=pos_embed_apply_fn, q_norm=deepcopy(q_norm),
                         k_norm=deepcopy(k_norm))
        if qkv_split:
            mixer = SelfAttentionQKV(
                q=nn.Linear(dim, head_dim * n_heads, bias=attn_bias),
                k=nn.Linear(dim, head_dim * kv_heads, bias=attn_bias),
                v=nn.Linear(dim, head_dim * kv_heads, bias=attn_bias),
                attention=core, out=nn.Linear(head_dim * n_heads, dim, bias=attn_bias),
                q_init=partial(kaiming_linear_), k_init=partial(kaiming_linear_),
                v_init=partial(kaiming_linear_), out_init=partial(kaiming_linear_, scale=out_scale),
                layer_type=layer_type)
        else:
            mixer = SelfAttention(
                qkv=nn.Linear(dim, head_dim * (n_heads + 2 * kv_heads), bias=attn_bias),
                attention=core, out=nn.Linear(head_dim * n_heads, dim, bias=attn_bias), qkv_split="llama",
                qkv_init=partial(kaiming_linear_), out_init=partial(kaiming_linear_, scale=out_scale),
                layer_type=layer_type)

    norm_post = norm
    if norm is None:
        norm = RMSNorm(dim, eps=rms_norm_epsilon, fast=fast_norm)
        norm_post = RMSNorm(dim, eps=rms_norm_epsilon, fast=fast_norm,
                            weight_init=partial(nn.init.constant_, val=out_scale))

    mixer_block = ResidualBlock(deepcopy(norm), mixer, post_norm=(deepcopy(norm_post) if post_norm else None))
    if not use_ffn:
        return mixer_block

    gated_act, base_act = call[get_activation](ffn_activation)
    if gated_ff_split:
        ff = GatedFeedForward(
            nn.Linear(dim, intermediate_size, bias=ffn_bias), nn.Linear(dim, intermediate_size, bias=ffn_bias),
            deepcopy(base_act), nn.Linear(intermediate_size, dim, bias=ffn_bias),
            linear_proj_init=partial(kaiming_linear_), linear_gate_init=partial(kaiming_linear_),
            linear_out_init=partial(kaiming_linear_, scale=out_scale))
    else:
        first = intermediate_size * 2 if base_act is not None else intermediate_size
        ff = FeedForward(nn.Linear(dim, first, bias=ffn_bias), deepcopy(gated_act),
                         nn.Linear(intermediate_size, dim, bias=ffn_bias),
                         linear1_init=partial(kaiming_linear_),
                         linear2_init=partial(kaiming_linear_, scale=out_scale))
    return TransformerEncoderBlock(
        mixer_block,
        ResidualBlock(deepcopy(norm), ff, post_norm=(deepcopy(norm_post) if post_norm else None)))


@config_fn
def get_n_res_blocks(layers):
    n = 0
    for layer in layers:
        n += get_value(layer, "n_layer", 1) * (2 if get_value(layer, "use_ffn", True) else 1)
    return n


@config_fn
def build_block(layer_id, layers, dim, intermediate_size, n_res_blocks, attn_kwargs=None, mamba2_kwargs=None,
                norm=None, pos_embed_apply_fn=None):
    blocks = []
    for layer in layers:
        for _ in range(get_value(layer, "n_layer", 1)):
            blocks.append(build_layer(
                layer_id=layer_id, dim=dim, intermediate_size=intermediate_size, n_res_blocks=n_res_blocks,
                seq_mixer=get_value(layer, "mixer", "attention"), attn_kwargs=attn_kwargs,
                mamba2_kwargs=mamba2_kwargs, use_ffn=get_value(layer, "use_ffn", True), norm=norm,
                pos_embed_apply_fn=pos_embed_apply_fn))
            layer_id += 1
    return HNetBlock(dim, blocks)


def build_hnet(arch, dims, intermediate_sizes, attn_kwargs, mamba2_kwargs, norm, pos_embeds, pos_embed_apply_fn,
               stage_idx=0, parent_n_res_blocks=0, dechunk_heads=1, dechunk_block_size=64):
    stage = dict(dim=dims[stage_idx], intermediate_size=intermediate_sizes[stage_idx],
                 attn_kwargs=get_stage_kwargs(attn_kwargs, stage_idx),
                 mamba2_kwargs=get_stage_kwargs(mamba2_kwargs, stage_idx), norm=norm,
                 pos_embed_apply_fn=pos_embed_apply_fn)
    if len(arch) == 1:
        layers = arch[0]
        return build_block(stage_idx, layers, n_res_blocks=parent_n_res_blocks + get_n_res_blocks(layers), **stage)

    encoder, inner, decoder = arch
    n_res_blocks = parent_n_res_blocks + get_n_res_blocks(encoder) + get_n_res_blocks(decoder)
    inner_arch = [inner] if is_layer_group(inner) else inner
    main = call[build_hnet](inner_arch, dims, intermediate_sizes, attn_kwargs, mamba2_kwargs, norm, pos_embeds,
                            pos_embed_apply_fn, stage_idx + 1, n_res_blocks, dechunk_heads, dechunk_block_size)
    if len(inner_arch) == 1:
        # an innermost block stack still gets its own stage wrapper (rotary table, width padding)
        main = HNet(dims[stage_idx + 1], stage_idx + 1, main, None, None, pos_embeds[stage_idx + 1],
                    dims[stage_idx])
    return HNet(dims[stage_idx], stage_idx, main,
                build_block(stage_idx, encoder, n_res_blocks=n_res_blocks, **stage),
                build_block(stage_idx, decoder, n_res_blocks=n_res_blocks, **stage),
                pos_embeds[stage_idx], dims[stage_idx - 1] if stage_idx > 0 else None,
                n_heads=dechunk_heads, block_size=dechunk_block_size)


@config_fn
def hnet(arch, dims, intermediate_sizes, pos_dims, attn_kwargs, mamba2_kwargs, vocab_size, context_len,
         pos_embed="rope", pos_embed_apply_fn=None, embedding=None, use_head=True, target_ratios=None,
         ratio_loss_weight=0.03):
    pos_embeds = [None] * len(dims)
    if isinstance(pos_embed, str) and pos_embed == "rope":
        pos_embeds = [RotaryEmbedding(pos_dim, context_len, use_fused=True) for pos_dim in pos_dims]
        pos_embed_apply_fn = partial(apply_rotary_emb, use_fused=True, inplace=True)
    if embedding is None:
        embedding = TextEmbedding(nn.Embedding(vocab_size, dims[0]), 0, embed_init=partial(kaiming_linear_))
    head = None
    if use_head:
        head = VocabParallelLinear(nn.Linear(dims[0], vocab_size, bias=False), linear_init=partial(kaiming_linear_))
    model = build_hnet(arch, dims, intermediate_sizes, attn_kwargs=attn_kwargs, mamba2_kwargs=mamba2_kwargs,
                       norm=None, pos_embeds=pos_embeds, pos_embed_apply_fn=pos_embed_apply_fn)
    return HNetDecoder(embedding=embedding, hnet=model, head=head, target_ratios=target_ratios,
                       ratio_loss_weight=ratio_loss_weight)
