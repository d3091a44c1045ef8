"""Move a training state dict into an inference model's layout (reference:
distributed/state_dict.py:5-38). Source tensors may be plain, DTensors, or parameter views
of the flat sharded buffers; targets are described by the inference model's (meta) state
dict. Tensor-parallel targets take their slice of the full tensor.
"""

from __future__ import annotations

import torch


def _full(t):
    if hasattr(t, "full_tensor"):
        return t.full_tensor()
    return t


def reshard_state_dict(source, target, device=None, dtype=None, tp_rank=0, tp_size=1, tp_plan=None,
                       in_place=False):
    """Returns {key: tensor} for every key of `target`. `tp_plan` maps key -> ("shard", dim) or
    ("shard_parts", dim, parts) for tensors the inference model holds a 1/tp_size slice of. With `in_place` the values are
    copied into `target`'s own tensors (which keep their addresses) and `target` is returned."""
    out = {}
    for key, ref in target.items():
        src_key = key
        if src_key not in source and "_orig_mod." in src_key:
            src_key = src_key.replace("_orig_mod.", "")
        if src_key not in source:
            alt = [k for k in source if k.replace("_orig_mod.", "") == src_key]
            if not alt:
                raise KeyError(f"state dict is missing {key!r}")
            src_key = alt[0]
        t = _full(source[src_key]).detach()
        if tp_plan and key in tp_plan and tp_size > 1:
            kind, dim = tp_plan[key][0], tp_plan[key][1]
            if kind == "shard":
                n = t.shape[dim] // tp_size
                t = t.narrow(dim, tp_rank * n, n)
            elif kind == "shard_parts":
                # consecutive blocks along `dim` (q | k | v rows) are each cut for this rank
                pieces, at = [], 0
                for n in tp_plan[key][2]:
                    step = n // tp_size
                    pieces.append(t.narrow(dim, at + tp_rank * step, step))
                    at += n
                t = torch.cat(pieces, dim)
        if in_place:
            if tuple(t.shape) != tuple(ref.shape):
                raise ValueError(f"shape mismatch for {key}: {tuple(t.shape)} vs {tuple(ref.shape)}")
            with torch.no_grad():
                ref.copy_(t)
            out[key] = ref
            continue
        want_dtype = dtype or (ref.dtype if ref.dtype.is_floating_point and not ref.is_meta else t.dtype)
        if ref.is_meta:
            want_dtype = dtype or t.dtype
        t = t.to(device=device if device is not None else t.device, dtype=want_dtype)
        # the engine owns its copy: training may overwrite the source while rollouts run
        if t.data_ptr() == source[src_key].data_ptr() if hasattr(source[src_key], "data_ptr") else False:
            t = t.clone()
        if tuple(t.shape) != tuple(ref.shape):
            raise ValueError(f"shape mismatch for {key}: {tuple(t.shape)} vs {tuple(ref.shape)}")
        out[key] = t.contiguous()
    return out
