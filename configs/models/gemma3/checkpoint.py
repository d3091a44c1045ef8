"""Hugging Face Gemma-3 (multimodal) checkpoint keys -> native keys."""

from ..checkpoint_maps import fuse_projections
from ..siglip2.checkpoint_vision import vision_weight_maps

_COL, _ROW, _REP = ("shard", 0), ("shard", 1), "replicate"
_LM = "language_model.model."

_LAYER = [
    ("input_layernorm", "self_attention.pre_norm", _REP), ("post_attention_layernorm", "self_attention.post_norm", _REP),
    ("pre_feedforward_layernorm", "ff.pre_norm", _REP), ("post_feedforward_layernorm", "ff.post_norm", _REP),
    ("self_attn.q_proj", "self_attention.module.q", _COL), ("self_attn.k_proj", "self_attention.module.k", _COL),
    ("self_attn.v_proj", "self_attention.module.v", _COL), ("self_attn.o_proj", "self_attention.module.out", _ROW),
    ("self_attn.q_norm", "self_attention.module.attention.q_norm", _REP),
    ("self_attn.k_norm", "self_attention.module.attention.k_norm", _REP),
    ("mlp.gate_proj", "ff.module.linear_gate", _COL), ("mlp.up_proj", "ff.module.linear_proj", _COL),
    ("mlp.down_proj", "ff.module.linear_out", _ROW),
]

weight_maps = vision_weight_maps("embedding.image_embedding.encoder.")
weight_maps.update({
    "multi_modal_projector.mm_soft_emb_norm": {"key": "embedding.image_embedding.soft_embed_norm",
                                               "placement": {"weight": _REP}},
    "multi_modal_projector": {"key": "embedding.image_embedding", "name_map": {"input_proj": "mm_input_projection_weight"},
                              "placement": {"input_proj": _REP}},
    _LM + "embed_tokens": {"key": "embedding.text_embedding.embed_input_ids", "placement": {"weight": _COL}},
    _LM + "norm": {"key": "post_blocks.module", "placement": {"weight": _REP}},
})
for _hf, _native, _place in _LAYER:
    weight_maps[_LM + "layers.#." + _hf] = {"key": "blocks.#." + _native, "placement": {"weight": _place}}


def to_halite_postprocess(config, state_dict):
    # keys already carry the split-MLP names; only q|k|v fusing may apply
    cfg = {"qkv_split": config.get("qkv_split", True) if hasattr(config, "get") else True, "gated_ff_split": True}
    out = fuse_projections(cfg, {k: v for k, v in state_dict.items()})
    return out
