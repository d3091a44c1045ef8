"""Hugging Face SigLIP2 vision-tower keys -> native encoder keys. `vision_weight_maps(prefix)`
places the encoder under a prefix when it is embedded in a larger model."""

_BOTH = {"weight": "replicate", "bias": "replicate"}

_LAYER = [
    ("layer_norm1", "self_attention.pre_norm"), ("layer_norm2", "ff.pre_norm"),
    ("self_attn.q_proj", "self_attention.module.q"), ("self_attn.k_proj", "self_attention.module.k"),
    ("self_attn.v_proj", "self_attention.module.v"), ("self_attn.out_proj", "self_attention.module.out"),
    ("mlp.fc1", "ff.module.linear1"), ("mlp.fc2", "ff.module.linear2"),
]


def vision_weight_maps(prefix=""):
    maps = {
        "vision_model.embeddings.patch_embedding": {"key": prefix + "embedding.patch_embedding", "placement": dict(_BOTH)},
        "vision_model.embeddings.position_embedding": {
            "key": prefix + "embedding.position_embedding", "name_map": {"pos_embed": "weight"},
            "placement": {"pos_embed": "replicate"}},
        "vision_model.post_layernorm": {"key": prefix + "post_blocks.module", "placement": dict(_BOTH)},
    }
    for hf, native in _LAYER:
        maps["vision_model.encoder.layers.#." + hf] = {"key": prefix + "blocks.#." + native, "placement": dict(_BOTH)}
    return maps


weight_maps = vision_weight_maps()


def to_halite_postprocess(config, state_dict):
    """A linear patch embedding stores the conv kernel flattened: [dim, 3, p, p] -> [dim, 3*p*p]."""
    get = (lambda k, d=None: config.get(k, d)) if hasattr(config, "get") else (lambda k, d=None: getattr(config, k, d))
    out = dict(state_dict)
    if not get("use_conv", True):
        for k, v in state_dict.items():
            if k.endswith("embedding.patch_embedding.weight") and v.ndim == 4:
                out[k] = v.flatten(1)
    return out
