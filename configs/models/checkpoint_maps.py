"""Weight-map builders for decoder checkpoints in Meta and Hugging Face layouts, and the
post-processing that fuses q|k|v and gate|up when the model is configured with fused
projections (reference: configs/models/llama/checkpoint.py, configs/models/qwen3/checkpoint.py)."""

import torch

from halite_b200.models.convert import get_matched_keys

_COL, _ROW, _REP = ("shard", 0), ("shard", 1), "replicate"

# (native sub-key, placement, Meta name, HF name)
_BLOCK = [
    ("self_attention.pre_norm", _REP, "attention_norm", "input_layernorm"),
    ("self_attention.module.q", _COL, "attention.wq", "self_attn.q_proj"),
    ("self_attention.module.k", _COL, "attention.wk", "self_attn.k_proj"),
    ("self_attention.module.v", _COL, "attention.wv", "self_attn.v_proj"),
    ("self_attention.module.out", _ROW, "attention.wo", "self_attn.o_proj"),
    ("ff.pre_norm", _REP, "ffn_norm", "post_attention_layernorm"),
    ("ff.module.linear_gate", _COL, "feed_forward.w1", "mlp.gate_proj"),
    ("ff.module.linear2", _ROW, "feed_forward.w2", "mlp.down_proj"),
    ("ff.module.linear1", _COL, "feed_forward.w3", "mlp.up_proj"),
]
_QK_NORM = [
    ("self_attention.module.attention.q_norm", _REP, None, "self_attn.q_norm"),
    ("self_attention.module.attention.k_norm", _REP, None, "self_attn.k_norm"),
]
_TOP = [
    ("embedding.embed_input_ids", _COL, "tok_embeddings", "model.embed_tokens"),
    ("post_blocks.module", _REP, "norm", "model.norm"),
    ("head.linear", _COL, "output", "lm_head"),
]


def decoder_weight_maps(style="hf", qk_norm=False, bias=False):
    col = 2 if style == "meta" else 3
    layer_prefix = "layers.#." if style == "meta" else "model.layers.#."
    maps = {}
    for native, place, *names in _TOP:
        maps[names[col - 2]] = {"key": native, "placement": {"weight": place}}
    for native, place, *names in _BLOCK + (_QK_NORM if qk_norm else []):
        name = names[col - 2]
        if name is None:
            continue
        placement = {"weight": place}
        if bias and place != _REP:
            placement["bias"] = place if place == _COL else _REP
        maps[layer_prefix + name] = {"key": "blocks.#." + native, "placement": placement}
    return maps


def fuse_projections(config, state_dict):
    """Native keys as converted (separate q, k, v, linear1, linear_gate, linear2) -> the layout
    the configured model expects: `qkv` when not `qkv_split`; `linear_proj`/`linear_out` names
    for the split gated MLP, or one `linear1 = [gate; up]` when fused."""
    get = (lambda k, d=None: config.get(k, d)) if hasattr(config, "get") else (lambda k, d=None: getattr(config, k, d))
    keys = list(state_dict)
    out, consumed = {}, set()
    pre = "blocks.#.self_attention.module."
    if not get("qkv_split", True):
        for attr in ("weight", "bias"):
            qs, fused = get_matched_keys(keys, pre + "q." + attr, pre + "qkv." + attr)
            ks = get_matched_keys(keys, pre + "k." + attr)
            vs = get_matched_keys(keys, pre + "v." + attr)
            for q, k, v, dst in zip(qs, ks, vs, fused):
                out[dst] = torch.cat((state_dict[q], state_dict[k], state_dict[v]), 0)
                consumed.update((q, k, v))
    ff = "blocks.#.ff.module."
    if get("gated_ff_split", True):
        for src, dst in (("linear1", "linear_proj"), ("linear2", "linear_out")):
            for attr in ("weight", "bias"):
                olds, news = get_matched_keys(keys, ff + src + "." + attr, ff + dst + "." + attr)
                for o, n in zip(olds, news):
                    out[n] = state_dict[o]
                    consumed.add(o)
    else:
        ups = get_matched_keys(keys, ff + "linear1.weight")
        gates = get_matched_keys(keys, ff + "linear_gate.weight")
        for up, gate in zip(ups, gates):
            out[up] = torch.cat((state_dict[gate], state_dict[up]), 0)
            consumed.update((up, gate))
    for k, v in state_dict.items():
        if k not in consumed and k not in out:
            out[k] = v
    return out


def unfuse_projections(config, state_dict):
    """Inverse of `fuse_projections`: the configured model's layout -> separate q, k, v,
    linear1 (up), linear_gate, linear2, which is what the weight maps name."""
    get = (lambda k, d=None: config.get(k, d)) if hasattr(config, "get") else (lambda k, d=None: getattr(config, k, d))
    out = {}
    for key, val in state_dict.items():
        if ".self_attention.module.qkv." in key:
            q_rows = get("n_heads") * get("head_dim")
            kv_rows = (get("n_key_value_heads") or get("n_heads")) * get("head_dim")
            q, k, v = torch.split(val, [q_rows, kv_rows, kv_rows], 0)
            for name, part in (("q", q), ("k", k), ("v", v)):
                out[key.replace(".qkv.", f".{name}.")] = part
        elif ".ff.module.linear_proj." in key:
            out[key.replace(".linear_proj.", ".linear1.")] = val
        elif ".ff.module.linear_out." in key:
            out[key.replace(".linear_out.", ".linear2.")] = val
        elif ".ff.module.linear1." in key and not get("gated_ff_split", True) and key.endswith("weight"):
            gate, up = torch.chunk(val, 2, 0)
            out[key.replace(".linear1.", ".linear_gate.")] = gate
            out[key] = up
        else:
            out[key] = val
    return out
