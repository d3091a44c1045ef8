"""Model zoo assembly: `transformer(...)` builds a decoder config out of small components,
`transformer_infer(...)` returns the patch list that rewrites such a config into its paged-KV
inference twin. Same keyword surface as the reference's configs/models/transformer.py
(`transformer`, `build_block`, `transformer_infer`, `use_flash_attention`,
`use_fused_linear_cross_entropy`), so experiment configs port by changing the import root.
"""

from copy import deepcopy
from functools import partial

from halite_b200.conf import annotate, call, config_fn, patch, patch_fn, select
from torch import nn

from halite_b200.nn.activation import GEGLU, SwiGLU
from halite_b200.nn.normalization import RMSNorm
from halite_b200.models.attention import Attention, SelfAttention, SelfAttentionQKV
from halite_b200.models.block import FusedTransformerEncoderBlock, ResidualBlock, TransformerEncoderBlock
from halite_b200.models.embedding import TextEmbedding
from halite_b200.models.feedforward import (FeedForward, FusedLinearCrossEntropy, GatedFeedForward,
                                            SequenceParallelWrapper, VocabParallelLinear)
from halite_b200.models.position import RotaryEmbedding, apply_rotary_emb
from halite_b200.models.transformer import TransformerDecoder

try:
    from halite_b200.infer.attention import InferSelfAttention, InferSelfAttentionQKV, PagedAttention
    from halite_b200.infer.block import InferTransformerEncoderBlock
    from halite_b200.infer.transformer import InferTransformerDecoder
except ImportError:
    pass

DEFAULT_INIT = partial(nn.init.kaiming_normal_, nonlinearity="linear")

ACTIVATIONS = {
    # name -> (module applied to a packed [gate | up] tensor, activation of the gate alone)
    "swiglu": (SwiGLU(), nn.SiLU()),
    "gelu_tanh": (nn.GELU(approximate="tanh"), None),
    "geglu_tanh": (GEGLU(approximate="tanh"), nn.GELU(approximate="tanh")),
}


@config_fn
def get_activation(activation):
    return ACTIVATIONS.get(activation)


@config_fn
def build_attention(layer_id, dim, n_heads, head_dim, n_key_value_heads, softcap, pos_embed_apply_fn,
                    attention_processor, attention_bias, is_causal, qkv_split, infer, q_norm, k_norm,
                    layer_type, init):
    kv_heads = n_key_value_heads if n_key_value_heads is not None else n_heads
    if infer is not None:
        core = PagedAttention(annotate("layer_id", layer_id), n_heads, head_dim,
                              n_key_value_heads=n_key_value_heads, apply_pos_emb_fn=pos_embed_apply_fn,
                              q_norm=deepcopy(q_norm), k_norm=deepcopy(k_norm))
    else:
        core = Attention(n_heads, head_dim, n_key_value_heads=n_key_value_heads, attn_drop=0,
                         apply_pos_emb_fn=pos_embed_apply_fn, processor=attention_processor,
                         softcap=softcap, is_causal=is_causal, q_norm=deepcopy(q_norm),
                         k_norm=deepcopy(k_norm))
    out = nn.Linear(head_dim * n_heads, dim, bias=attention_bias)
    if qkv_split:
        cls = InferSelfAttentionQKV if infer is not None else SelfAttentionQKV
        return cls(
            q=nn.Linear(dim, head_dim * n_heads, bias=attention_bias),
            k=nn.Linear(dim, head_dim * kv_heads, bias=attention_bias),
            v=nn.Linear(dim, head_dim * kv_heads, bias=attention_bias),
            attention=core, out=out, q_init=init, k_init=init, v_init=init, out_init=init,
            layer_type=layer_type)
    cls = InferSelfAttention if infer is not None else SelfAttention
    return cls(qkv=nn.Linear(dim, head_dim * (n_heads + 2 * kv_heads), bias=attention_bias),
               attention=core, out=out, qkv_split="llama", qkv_init=init, out_init=init,
               layer_type=layer_type)


@config_fn
def build_ff(dim, intermediate_size, ffn_bias, ffn_activation, gated_ff_split, init):
    packed_act, gate_act = call[get_activation](ffn_activation)
    if gated_ff_split:
        return GatedFeedForward(
            nn.Linear(dim, intermediate_size, bias=ffn_bias),
            nn.Linear(dim, intermediate_size, bias=ffn_bias),
            deepcopy(gate_act),
            nn.Linear(intermediate_size, dim, bias=ffn_bias),
            linear_proj_init=init, linear_gate_init=init, linear_out_init=init)
    hidden = intermediate_size * 2 if gate_act is not None else intermediate_size
    return FeedForward(nn.Linear(dim, hidden, bias=ffn_bias), deepcopy(packed_act),
                       nn.Linear(intermediate_size, dim, bias=ffn_bias),
                       linear1_init=init, linear2_init=init)


@config_fn
def build_block(layer_id, dim, n_heads, head_dim, n_layers, intermediate_size, n_key_value_heads=None,
                softcap=0.0, norm=None, rms_norm_epsilon=1e-6, post_norm=False, pos_embed_apply_fn=None,
                attention_processor="auto", attention_bias=False, is_causal=True, qkv_split=False,
                ffn_bias=False, ffn_activation="swiglu", gated_ff_split=False, fast_norm=False,
                infer: str | None = None, q_norm=None, k_norm=None, layer_type=None, init=None):
    init = init if init is not None else DEFAULT_INIT
    if norm is None:
        norm = RMSNorm(dim, eps=rms_norm_epsilon, fast=fast_norm)
        norm_post = RMSNorm(dim, eps=rms_norm_epsilon, fast=fast_norm,
                            weight_init=partial(nn.init.constant_, val=1 / (n_layers ** 0.5)))
    else:
        norm_post = norm
    attention = call[build_attention](layer_id, dim, n_heads, head_dim, n_key_value_heads, softcap,
                                      pos_embed_apply_fn, attention_processor, attention_bias, is_causal,
                                      qkv_split, infer, q_norm, k_norm, layer_type, init)
    ff = call[build_ff](dim, intermediate_size, ffn_bias, ffn_activation, gated_ff_split, init)
    block_cls = InferTransformerEncoderBlock if infer is not None else TransformerEncoderBlock
    return block_cls(
        ResidualBlock(deepcopy(norm), attention, post_norm=deepcopy(norm_post) if post_norm else None),
        ResidualBlock(deepcopy(norm), ff, post_norm=deepcopy(norm_post) if post_norm else None))


@config_fn
def transformer(vocab_size, dim, n_heads, head_dim, n_layers, intermediate_size, context_len,
                n_key_value_heads=None, pos_embed="rope", pos_embed_apply_fn=None, softcap=0.0,
                is_causal=True, norm=None, rms_norm_epsilon=1e-6, post_norm=False,
                attention_processor="auto", attention_bias=False, flex_attention_processor=None,
                qkv_split=False, gated_ff_split=False, ffn_bias=False, ffn_activation="swiglu",
                infer: str | None = None, embedding=None, q_norm=None, k_norm=None, use_head=True,
                tie_embeds=False, layer_types=None, init=None):
    init = init if init is not None else DEFAULT_INIT
    fast_norm = attention_processor == "flash_attn"
    if isinstance(pos_embed, str) and pos_embed == "rope":
        pos_embed = RotaryEmbedding(head_dim, context_len)
        pos_embed_apply_fn = partial(apply_rotary_emb)
    blocks = [
        call[build_block](
            i, dim, n_heads, head_dim, n_layers, intermediate_size, n_key_value_heads, softcap, norm,
            rms_norm_epsilon, post_norm, pos_embed_apply_fn, attention_processor, attention_bias,
            is_causal, qkv_split, ffn_bias, ffn_activation, gated_ff_split, fast_norm, infer=infer,
            q_norm=q_norm, k_norm=k_norm,
            layer_type=layer_types[i] if layer_types is not None else None, init=init)
        for i in range(n_layers)
    ]
    if embedding is None:
        embedding = TextEmbedding(nn.Embedding(vocab_size, dim), 0, embed_init=init)
    head = None
    if use_head:
        head = VocabParallelLinear(nn.Linear(dim, vocab_size, bias=False), linear_init=init)
    if norm is None:
        norm = RMSNorm(dim, eps=rms_norm_epsilon, fast=fast_norm)
    decoder_cls = InferTransformerDecoder if infer is not None else TransformerDecoder
    return decoder_cls(embedding=embedding, pos_embed=pos_embed, blocks=blocks,
                       post_blocks=SequenceParallelWrapper(norm), head=head, tie_embeds=tie_embeds,
                       use_position_ids=True, attention_processor=attention_processor,
                       flex_attention_processor=flex_attention_processor)


def _infer_patches(qkv_split):
    """Patch list turning a training decoder config into the paged-KV inference decoder."""
    patches = [
        patch_fn.select().instance(Attention).map_instance(
            PagedAttention, layer_id=0, n_heads="$n_heads", head_dim="$head_dim",
            n_key_value_heads="$n_key_value_heads", apply_pos_emb_fn="$apply_pos_emb_fn",
            q_norm="$q_norm", k_norm="$k_norm", softcap="$softcap").chain(),
        patch_fn.select().instance(PagedAttention).at("layer_id").set_sequence("$index").chain(),
    ]
    if qkv_split:
        patches.append(patch_fn.select().instance(SelfAttentionQKV).map_instance(
            InferSelfAttentionQKV, q="$q", k="$k", v="$v", attention="$attention", out="$out",
            q_init="$q_init", k_init="$k_init", v_init="$v_init", out_init="$out_init",
            scaler="$scaler", q_norm="$q_norm", k_norm="$k_norm").chain())
    else:
        patches.append(patch_fn.select().instance(SelfAttention).map_instance(
            InferSelfAttention, qkv="$qkv", attention="$attention", out="$out", qkv_split="llama",
            qkv_init="$qkv_init", out_init="$out_init", scaler="$scaler").chain())
    patches += [
        patch_fn.select().instance(TransformerEncoderBlock).map_instance(
            InferTransformerEncoderBlock, self_attention="$self_attention", ff="$ff").chain(),
        patch_fn.select().instance(TransformerDecoder).map_instance(
            InferTransformerDecoder, embedding="$embedding", pos_embed="$pos_embed", blocks="$blocks",
            post_blocks="$post_blocks", head="$head", tie_embeds="$tie_embeds",
            use_position_ids="$use_position_ids", attention_processor="$attention_processor").chain(),
    ]
    return patches


@config_fn
def transformer_infer(vocab_size=None, dim=None, n_heads=None, head_dim=None, n_layers=None,
                      intermediate_size=None, context_len=None, qkv_split=False,
                      infer: str | None = None, **unused):
    if infer is None:
        return partial(patch, patches=())
    return partial(patch, patches=_infer_patches(qkv_split))


# the multi-process engine of the reference shares the in-process engine's model classes here
transformer_tokainfer = transformer_infer


@config_fn
def use_flex_attention(model_conf):
    return select(model_conf).instance(Attention).update_dict(dict(processor="flex"))


@config_fn
def use_flash_attention(model_conf):
    return select(model_conf).instance(Attention).update_dict(dict(processor="flash_attn"))


@config_fn
def use_fused_residual(model_conf):
    """Pre-norm blocks that hand the un-normalised residual stream to the next norm, so every
    residual add runs inside the following RMSNorm kernel (forward and backward)."""
    return select(model_conf).instance(TransformerEncoderBlock).map(
        lambda x: FusedTransformerEncoderBlock(x.self_attention, x.ff))


@config_fn
def use_fused_linear_cross_entropy(model_conf, ignore_index=-100, z_loss=0):
    return select(model_conf).instance(VocabParallelLinear).map(
        lambda x: FusedLinearCrossEntropy(x.linear, x.get("linear_init"), ignore_index=ignore_index,
                                          z_loss=z_loss))
