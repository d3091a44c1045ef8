"""Checkpoint conversion between foreign layouts (Meta, Hugging Face) and this package's
state-dict keys (reference: transformers/convert.py:10-268).

A weight map is `{foreign_prefix: {"key": native_prefix, "placement": {attr: "replicate" |
("shard", dim)}, "name_map": {native_attr: foreign_attr}}}` with `#` standing for a layer
number. Patterns are compiled once into `KeyRule`s; both directions are implemented (the
reference leaves the export direction as a stub).
"""

from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Any, Callable

import torch

from halite_b200.conf import instantiate

Checkpoint = dict


def get_find_pattern(pattern: str, attr=None, ensure_ending=True):
    """Regex for a `#` pattern (+ optional attribute suffix) and its number of wildcards."""
    count = pattern.count("#")
    regex = re.escape(pattern).replace(r"\#", "([0-9]+)")
    if attr is not None:
        regex += r"\." + re.escape(attr)
    if ensure_ending:
        regex += "$"
    return regex, count


def get_replace_pattern(pattern: str, count: int):
    for i in range(count):
        pattern = pattern.replace("#", f"\\{i + 1}", 1)
    return pattern


def get_matched_keys(keys, pattern: str, replace_pattern=None):
    """Keys matching `pattern`, sorted; with `replace_pattern` also the rewritten keys."""
    regex, count = get_find_pattern(pattern)
    rx = re.compile(regex)
    found = {}
    for key in keys:
        m = rx.search(key)
        if m is None:
            continue
        src = m.group(0)
        found[src] = rx.sub(get_replace_pattern(replace_pattern, count), src) if replace_pattern is not None else src
    ordered = sorted(found.items(), key=lambda kv: _natural(kv[0]))
    if replace_pattern is not None:
        return tuple(zip(*ordered)) if ordered else ((), ())
    return tuple(k for k, _ in ordered)


def _natural(key):
    return [int(t) if t.isdigit() else t for t in re.split(r"(\d+)", key)]


@dataclass
class KeyRule:
    foreign: re.Pattern
    native: re.Pattern
    to_native: str
    to_foreign: str
    attr_native: str
    attr_foreign: str
    placement: Any


def compile_rules(weight_maps) -> list[KeyRule]:
    rules = []
    for foreign, spec in weight_maps.items():
        names = spec.get("name_map", {})
        for attr, placement in spec.get("placement", {"weight": "replicate"}).items():
            f_attr = names.get(attr, attr)
            f_rx, n = get_find_pattern(foreign, f_attr)
            n_rx, _ = get_find_pattern(spec["key"], attr)
            rules.append(KeyRule(re.compile("^" + f_rx), re.compile("^" + n_rx),
                                 get_replace_pattern(spec["key"], n) + "." + attr,
                                 get_replace_pattern(foreign, n) + "." + f_attr, attr, f_attr, placement))
    return rules


def convert_state_dict(state_dict, mapping, reverse=False):
    """Rename keys foreign -> native (or back with `reverse`); unmatched keys are dropped."""
    rules = compile_rules(mapping)
    out = {}
    for key, tensor in state_dict.items():
        for r in rules:
            rx, repl = (r.native, r.to_foreign) if reverse else (r.foreign, r.to_native)
            if rx.match(key):
                out[rx.sub(repl, key)] = tensor
                break
    return out


@dataclass
class Policy:
    weight_maps: dict
    to_halite_preprocess: Callable | None = None
    to_halite_postprocess: Callable | None = None
    from_halite_preprocess: Callable | None = None
    from_halite_postprocess: Callable | None = None

    @classmethod
    def from_pydantic(cls, config):
        def hook(name):
            val = config.get(name) if hasattr(config, "get") else getattr(config, name, None)
            if val is None:
                return None
            return val if callable(val) and not isinstance(val, dict) else instantiate(val)

        maps = config["weight_maps"] if hasattr(config, "__getitem__") else config.weight_maps
        return cls(weight_maps=maps, **{n: hook(n) for n in
                                        ("to_halite_preprocess", "to_halite_postprocess",
                                         "from_halite_preprocess", "from_halite_postprocess")})


def extract_placement(weight_maps, mode="to_halite"):
    out = {}
    for foreign, spec in weight_maps.items():
        if "placement" in spec:
            out[spec["key"] if mode == "to_halite" else foreign] = spec["placement"]
    return out


def unshard_tensor(state_dicts, key, placement):
    """Assemble one tensor from the tensor-parallel shards that carry `key`."""
    holders = [sd for sd in state_dicts if key in sd]
    if placement == "replicate" or len(holders) == 1:
        return holders[0][key]
    if not (isinstance(placement, (tuple, list)) and len(placement) == 2):
        raise ValueError("placement must be 'replicate' or ('shard', dim)")
    return torch.cat([sd[key] for sd in holders], placement[1])


def shard_tensor(tensor, placement, n_shards):
    if placement == "replicate" or n_shards == 1:
        return [tensor] * n_shards
    return list(torch.chunk(tensor, n_shards, placement[1]))


def convert_to_halite(state_dicts, model_config, policy: Policy):
    if not isinstance(state_dicts, (list, tuple)):
        state_dicts = [state_dicts]
    renamed = [convert_state_dict(sd, policy.weight_maps) for sd in state_dicts]
    if policy.to_halite_preprocess is not None:
        renamed = [policy.to_halite_preprocess(model_config, sd) for sd in renamed]
    rules = compile_rules(policy.weight_maps)
    merged = {}
    for sd in renamed:
        for key in sd:
            if key in merged:
                continue
            rule = next((r for r in rules if r.native.match(key)), None)
            if rule is not None:
                merged[key] = unshard_tensor(renamed, key, rule.placement)
    if policy.to_halite_postprocess is not None:
        merged = policy.to_halite_postprocess(model_config, merged)
    return merged


def convert_from_halite(state_dict, model_config, policy: Policy, n_shards: int = 1):
    """Native -> foreign keys; with `n_shards > 1` returns one state dict per tensor-parallel
    shard, cut along each weight's placement."""
    if policy.from_halite_preprocess is not None:
        state_dict = policy.from_halite_preprocess(model_config, state_dict)
    rules = compile_rules(policy.weight_maps)
    outs = [{} for _ in range(n_shards)]
    for key, tensor in state_dict.items():
        rule = next((r for r in rules if r.native.match(key)), None)
        if rule is None:
            continue
        target = rule.native.sub(rule.to_foreign, key)
        for sd, piece in zip(outs, shard_tensor(tensor, rule.placement, n_shards)):
            sd[target] = piece
    if policy.from_halite_postprocess is not None:
        outs = [policy.from_halite_postprocess(model_config, sd) for sd in outs]
    return outs[0] if n_shards == 1 else outs


def convert_checkpoint(state_dicts, model_config, policy, mode="to_halite", **kwargs):
    if not isinstance(policy, Policy):
        policy = Policy.from_pydantic(policy)
    if mode == "to_halite":
        return convert_to_halite(state_dicts, model_config, policy)
    if mode == "from_halite":
        return convert_from_halite(state_dicts, model_config, policy, **kwargs)
    raise ValueError(f"unsupported mode: {mode}, supported modes: to_halite, from_halite")
