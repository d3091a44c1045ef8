"""Small collective helpers and an extra-process-group constructor
(reference: distributed/__init__.py:14-118)."""

from __future__ import annotations

import socket
from datetime import timedelta

import torch
import torch.distributed as dist


def all_reduce_mean(tensor, group=None, world_size=None):
    dist.all_reduce(tensor, group=group)
    return tensor / (world_size if world_size is not None else dist.get_world_size(group))


def all_reduce_flag(flag, group=None, device="cpu"):
    """True on every rank when any rank passes True."""
    t = torch.tensor(float(bool(flag)), dtype=torch.float32, device=device)
    dist.all_reduce(t, group=group, op=dist.ReduceOp.MAX)
    return bool(t.item() > 0)


def find_local_ip():
    try:
        return socket.gethostbyname(socket.getfqdn())
    except OSError:
        return "127.0.0.1"


def find_free_port():
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("", 0))
        return s.getsockname()[1]


def init_custom_process_group(backend=None, init_method=None, timeout=None, world_size=-1, rank=-1,
                              device_id=None, store=None, group_name="custom", pg_options=None):
    """A process group with its own rendezvous, independent of the default group: used to join
    a trainer job and a separately launched generator job for weight broadcast."""
    from torch.distributed import distributed_c10d as c10d

    if store is not None and init_method is not None:
        raise ValueError("give either a store or an init_method, not both")
    timeout = timeout or c10d.default_pg_timeout
    if isinstance(timeout, (int, float)):
        timeout = timedelta(seconds=timeout)
    if store is None:
        rendezvous = c10d.rendezvous(init_method or "env://", rank, world_size, timeout=timeout)
        store, rank, world_size = next(rendezvous)
        store.set_timeout(timeout)
        store = c10d.PrefixStore(group_name, store)
    elif world_size <= 0 or rank < 0:
        raise ValueError("a store needs an explicit world_size and rank")
    be = c10d.Backend(backend) if backend else c10d.Backend("undefined")
    pg, _ = c10d._new_process_group_helper(world_size, rank, [], be, store, group_name=group_name,
                                           backend_options=pg_options, device_id=device_id, timeout=timeout)
    c10d._world.pg_group_ranks[pg] = {i: i for i in range(world_size)}
    return pg


from .checkpoint import CheckpointManager, load_checkpoint  # noqa: E402
from .managers import LRSchedulerManager, ModelManager, OptimizerManager  # noqa: E402

__all__ = ["all_reduce_mean", "all_reduce_flag", "find_local_ip", "find_free_port", "init_custom_process_group",
           "CheckpointManager", "load_checkpoint", "ModelManager", "OptimizerManager", "LRSchedulerManager"]
