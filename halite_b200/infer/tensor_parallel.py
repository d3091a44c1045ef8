"""Tensor parallelism for the inference modules (reference: the TP plans of infer/attention.py
and the tokainfer TP set-up, tokainfer/utils.py:397-412).

`apply_infer_tp(model, tp_rank, tp_size, group)` turns every attention and feed-forward module of
an `InferTransformerDecoder` into its rank's slice:

    q / k / v, up / gate   column-parallel: the rank keeps the rows of its heads / hidden units
    out, down              row-parallel: the rank keeps its input columns; partial results are
                           summed over the group right after the projection
    embedding, norms, head replicated

KV pages then hold only the rank's KV heads (the pool is sized with `ModelConfig.tp_size`). Every
rank of the group runs the same scheduler on the same requests; the sampler is seeded
identically, and an all-reduce returns bitwise-identical sums on every rank, so the ranks take
the same decisions without talking about them.

`tp_plan(model)` maps state-dict keys to ("shard", dim): what `reshard_state_dict` and the fused
reshard kernel (`parallel/reshard.py`) need to cut a full tensor down to this rank's part.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch import nn


@dataclass
class InferTP:
    rank: int
    size: int
    group: object = None

    def all_reduce(self, x):
        if self.size > 1:
            dist.all_reduce(x, group=self.group)
        return x


def _slice_linear(lin: nn.Linear, dim: int, rank: int, size: int, parts=None):
    """Replace `lin.weight` by this rank's slice along `dim` (meta tensors stay meta). `parts` splits
    dim 0 into consecutive blocks that are each cut separately (q | k | v rows of a packed
    projection)."""
    w = lin.weight
    if parts is None:
        parts = [w.shape[dim]]
    pieces, at = [], 0
    for n in parts:
        if n % size:
            raise ValueError(f"cannot split {n} rows / columns over {size} tensor-parallel ranks")
        step = n // size
        pieces.append(w.narrow(dim, at + rank * step, step))
        at += n
    new = pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim)
    lin.weight = nn.Parameter(new.contiguous() if not new.is_meta else torch.empty(new.shape, dtype=w.dtype, device="meta"),
                              requires_grad=False)
    if dim == 0:
        lin.out_features = lin.weight.shape[0]
        if lin.bias is not None:
            b = lin.bias
            bp, at = [], 0
            for n in parts:
                step = n // size
                bp.append(b.narrow(0, at + rank * step, step))
                at += n
            nb = bp[0] if len(bp) == 1 else torch.cat(bp, 0)
            lin.bias = nn.Parameter(nb.contiguous() if not nb.is_meta else torch.empty(nb.shape, dtype=b.dtype, device="meta"),
                                    requires_grad=False)
    else:
        lin.in_features = lin.weight.shape[1]


def apply_infer_tp(model, tp_rank: int, tp_size: int, group=None):
    """Shard `model` (an inference decoder, usually still on the meta device) in place. Returns the
    plan {state-dict key: ("shard", dim) or ("shard_parts", dim, parts)}."""
    from halite_b200.infer.attention import InferSelfAttention, InferSelfAttentionQKV
    from halite_b200.models.feedforward import FeedForward, GatedFeedForward

    if tp_size <= 1:
        return {}
    tp = InferTP(tp_rank, tp_size, group)
    plan = {}
    names = {id(m): n for n, m in model.named_modules()}

    def key(mod, sub):
        return f"{names[id(mod)]}.{sub}.weight"

    def also_bias(mod, sub):
        # a column-parallel projection's bias is cut like its weight's rows
        if getattr(getattr(mod, sub), "bias", None) is not None:
            entry = plan[key(mod, sub)]
            plan[f"{names[id(mod)]}.{sub}.bias"] = (entry[0], 0) + tuple(entry[2:])

    for mod in list(model.modules()):
        if isinstance(mod, InferSelfAttentionQKV):
            a = mod.attention
            if a.n_heads % tp_size or a.kv_heads % tp_size:
                raise ValueError("head counts must divide by the tensor-parallel size")
            for sub in ("q", "k", "v"):
                _slice_linear(getattr(mod, sub), 0, tp_rank, tp_size)
                plan[key(mod, sub)] = ("shard", 0)
                also_bias(mod, sub)
            _slice_linear(mod.out, 1, tp_rank, tp_size)
            plan[key(mod, "out")] = ("shard", 1)
            a.n_key_value_heads = a.kv_heads // tp_size
            a.n_heads //= tp_size
            mod._infer_tp = tp
        elif isinstance(mod, InferSelfAttention):
            a = mod.attention
            H, Hk, D = a.n_heads, a.kv_heads, a.head_dim
            if H % tp_size or Hk % tp_size:
                raise ValueError("head counts must divide by the tensor-parallel size")
            if mod.qkv_split == "megatron":
                _slice_linear(mod.qkv, 0, tp_rank, tp_size)          # kv groups are contiguous
                plan[key(mod, "qkv")] = ("shard", 0)
            else:
                parts = [H * D, Hk * D, Hk * D]
                _slice_linear(mod.qkv, 0, tp_rank, tp_size, parts)
                plan[key(mod, "qkv")] = ("shard_parts", 0, parts)
            also_bias(mod, "qkv")
            _slice_linear(mod.out, 1, tp_rank, tp_size)
            plan[key(mod, "out")] = ("shard", 1)
            a.n_key_value_heads = Hk // tp_size
            a.n_heads = H // tp_size
            mod._infer_tp = tp
        elif isinstance(mod, GatedFeedForward):
            for sub in ("linear_proj", "linear_gate"):
                _slice_linear(getattr(mod, sub), 0, tp_rank, tp_size)
                plan[key(mod, sub)] = ("shard", 0)
                also_bias(mod, sub)
            _slice_linear(mod.linear_out, 1, tp_rank, tp_size)
            plan[key(mod, "linear_out")] = ("shard", 1)
            mod._infer_tp = tp
        elif isinstance(mod, FeedForward):
            w = mod.linear1.weight
            gated = hasattr(mod.activation, "gate_first") or type(mod.activation).__name__ in ("SwiGLU", "GEGLU")
            parts = [w.shape[0] // 2, w.shape[0] // 2] if gated else None
            _slice_linear(mod.linear1, 0, tp_rank, tp_size, parts)
            plan[key(mod, "linear1")] = ("shard_parts", 0, parts) if parts else ("shard", 0)
            also_bias(mod, "linear1")
            _slice_linear(mod.linear2, 1, tp_rank, tp_size)
            plan[key(mod, "linear2")] = ("shard", 1)
            mod._infer_tp = tp
    model._infer_tp = tp
    model._infer_tp_plan = plan
    return plan


def row_parallel_linear(module, x, linear):
    """`linear(x)` for a projection whose input columns are split over the ranks: partial product,
    sum over the group, bias once."""
    from halite_b200 import ops

    tp = getattr(module, "_infer_tp", None)
    if tp is None or tp.size == 1:
        return ops.linear(x, linear.weight, linear.bias)
    y = ops.linear(x, linear.weight, None)
    tp.all_reduce(y)
    if linear.bias is not None:
        y = y + linear.bias
    return y
