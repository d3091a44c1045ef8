"""Collective wrappers used by the FSDP / TP layers, with Gloo fallbacks for the CPU tests
(Gloo lacks reduce_scatter and the AVG reduction)."""

from __future__ import annotations

import torch
import torch.distributed as dist


def _is_gloo(group):
    try:
        return dist.get_backend(group) == "gloo"
    except Exception:
        return False


def all_gather_flat(out: torch.Tensor, shard: torch.Tensor, group, async_op=False):
    """out[ws * n] <- concat over ranks of shard[n]; `shard` may be the matching slice of `out`."""
    if group is None:
        if out.data_ptr() != shard.data_ptr():
            out.copy_(shard)
        return None
    return dist.all_gather_into_tensor(out, shard, group=group, async_op=async_op)


def reduce_scatter_flat(out: torch.Tensor, full: torch.Tensor, group, average=True, async_op=False):
    """out[n] <- (mean | sum) over ranks of full[rank * n : (rank + 1) * n]."""
    if group is None:
        if out.data_ptr() != full.data_ptr():
            out.copy_(full[: out.numel()])
        return None
    ws = dist.get_world_size(group)
    if _is_gloo(group):
        dist.all_reduce(full, group=group)
        r = dist.get_rank(group)
        n = out.numel()
        out.copy_(full[r * n:(r + 1) * n])
        if average:
            out.div_(ws)
        return None
    op = dist.ReduceOp.AVG if average else dist.ReduceOp.SUM
    return dist.reduce_scatter_tensor(out, full, op=op, group=group, async_op=async_op)


def all_reduce(t: torch.Tensor, group, average=False, op=None, async_op=False):
    if group is None:
        return None
    if op is not None:
        return dist.all_reduce(t, op=op, group=group, async_op=async_op)
    if average and _is_gloo(group):
        dist.all_reduce(t, group=group)
        t.div_(dist.get_world_size(group))
        return None
    return dist.all_reduce(t, op=dist.ReduceOp.AVG if average else dist.ReduceOp.SUM, group=group,
                           async_op=async_op)
