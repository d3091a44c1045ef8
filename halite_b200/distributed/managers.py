"""`Stateful` adapters between the training objects and `torch.distributed.checkpoint`
(reference: distributed/managers.py:16-110).

Model: parameters are always resident in full inside the sharding layer's flat buffers, so
the model state is a dict of full tensors under the reference's key names; DCP writes each
replicated tensor once. Optimizer: the fp32 master / moment shards are exposed as DTensors
sharded on dim 0 over the data-parallel group, which lets DCP reshard them when the world size
changes between save and load.
"""

from __future__ import annotations

from collections.abc import Sequence

import torch
import torch.distributed as dist
from torch import nn
from torch.distributed.checkpoint.stateful import Stateful


def _clean(key: str) -> str:
    return key.replace("_orig_mod.", "")


class ModelManager(Stateful):
    def __init__(self, model):
        self.models = [model] if isinstance(model, nn.Module) else list(model)

    def state_dict(self):
        out = {}
        for m in self.models:
            for k, v in m.state_dict().items():
                out[_clean(k)] = v.detach()
        return out

    def load_state_dict(self, state_dict):
        for m in self.models:
            own = m.state_dict()
            with torch.no_grad():
                for k, v in own.items():
                    src = state_dict.get(_clean(k))
                    if src is not None and src.data_ptr() != v.data_ptr():
                        v.copy_(src)
            fsdp = getattr(m, "_hb_fsdp", None)
            if fsdp is not None:
                for u in fsdp.units:
                    if u.master is not None:
                        u.master.copy_(u.param_shard())


def _as_dtensor(shard, group):
    if group is None or dist.get_world_size(group) == 1:
        return shard
    from torch.distributed.device_mesh import DeviceMesh
    from torch.distributed.tensor import DTensor, Shard

    mesh = DeviceMesh.from_group(group, shard.device.type)
    return DTensor.from_local(shard, mesh, [Shard(0)], run_check=False)


def _to_local(t):
    return t.to_local() if hasattr(t, "to_local") else t


class OptimizerManager(Stateful):
    def __init__(self, model_parts, optimizers=None, optimizer_fn=None):
        self.model_parts = list(model_parts) if isinstance(model_parts, Sequence) else [model_parts]
        if optimizers is None:
            optimizers = [optimizer_fn(p.parameters()) for p in self.model_parts]
        self.optimizers = list(optimizers) if isinstance(optimizers, Sequence) else [optimizers]

    def step(self):
        for o in self.optimizers:
            o.step()

    def zero_grad(self):
        for o in self.optimizers:
            o.zero_grad()

    def state_dict(self):
        out = {}
        for i, opt in enumerate(self.optimizers):
            prefix = "" if len(self.optimizers) == 1 else f"{i}."
            if hasattr(opt, "fsdp"):
                group = opt.fsdp.shard_group
                for k, v in opt.state_dict().items():
                    if isinstance(v, torch.Tensor):
                        out[prefix + k] = _as_dtensor(v, group)
                    elif k == "step":
                        out[prefix + k] = torch.tensor(v)
                    else:
                        out[prefix + k] = v
            else:
                sd = opt.state_dict()
                for pid, st in sd["state"].items():
                    for name, val in st.items():
                        out[f"{prefix}state.{pid}.{name}"] = val
                out[prefix + "param_groups"] = sd["param_groups"]
        return out

    def extend_load_template(self, template, saved):
        """Add to `template` (this manager's `state_dict()` of a FRESH optimizer) every entry the
        checkpoint holds and the fresh optimizer has not created yet. A torch optimizer builds its
        per-parameter state (moments, preconditioner factors, step counts) lazily in its first
        `step()`, so the fresh template has none of those keys and a load that only asks for the
        template's keys would silently restart them from zero. `saved` maps this group's saved
        keys to their checkpoint metadata (tensor entries carry `size` and `properties.dtype`)."""
        for i, opt in enumerate(self.optimizers):
            if hasattr(opt, "fsdp"):
                continue
            prefix = "" if len(self.optimizers) == 1 else f"{i}."
            device = torch.device("cpu")
            for g in opt.param_groups:
                if g["params"]:
                    device = g["params"][0].device
                    break
            for key, md in saved.items():
                if not key.startswith(prefix + "state.") or key in template:
                    continue
                if hasattr(md, "size") and hasattr(md, "properties"):
                    size = tuple(md.size)
                    # scalar entries (step counters) stay on the host, where torch keeps them
                    where = device if len(size) > 0 and md.size.numel() > 1 else torch.device("cpu")
                    template[key] = torch.empty(size, dtype=md.properties.dtype, device=where)
                else:
                    template[key] = None       # a pickled object: the loader replaces the value

    def load_state_dict(self, state_dict):
        for i, opt in enumerate(self.optimizers):
            prefix = "" if len(self.optimizers) == 1 else f"{i}."
            if hasattr(opt, "fsdp"):
                flat = {}
                for k, v in state_dict.items():
                    if k.startswith(prefix):
                        key = k[len(prefix):]
                        flat[key] = _to_local(v) if isinstance(v, torch.Tensor) else v
                if "step" in flat and isinstance(flat["step"], torch.Tensor):
                    flat["step"] = int(flat["step"])
                opt.load_state_dict(flat)
            else:
                sd = opt.state_dict()
                state = {pid: dict(st) for pid, st in sd["state"].items()}
                head = prefix + "state."
                for key, val in state_dict.items():
                    if not key.startswith(head):
                        continue
                    pid, _, name = key[len(head):].partition(".")
                    state.setdefault(int(pid), {})[name] = val
                # list-valued entries (one preconditioner factor per dimension) are stored element
                # by element under `name.index`: put them back together
                for st in state.values():
                    parts = {}
                    for name in [n for n in st if "." in n and n.rpartition(".")[2].isdigit()]:
                        base, _, idx = name.rpartition(".")
                        parts.setdefault(base, {})[int(idx)] = st.pop(name)
                    for base, items in parts.items():
                        st[base] = [items[j] for j in sorted(items)]
                sd["state"] = state
                if prefix + "param_groups" in state_dict:
                    saved_groups = state_dict[prefix + "param_groups"]
                    if len(saved_groups) == len(sd["param_groups"]):
                        for cur, old in zip(sd["param_groups"], saved_groups):
                            cur.update({k: v for k, v in old.items() if k != "params"})
                opt.load_state_dict(sd)


class LRSchedulerManager:
    def __init__(self, optimizers, schedulers=None, scheduler_fn=None):
        if isinstance(optimizers, OptimizerManager):
            optimizers = optimizers.optimizers
        optimizers = list(optimizers) if isinstance(optimizers, Sequence) else [optimizers]
        if schedulers is None:
            schedulers = [scheduler_fn(o) for o in optimizers]
        self.schedulers = list(schedulers) if isinstance(schedulers, Sequence) else [schedulers]

    def step(self):
        for s in self.schedulers:
            s.step()

    def get_state_dict(self):
        if len(self.schedulers) == 1:
            return {"lr_scheduler": self.schedulers[0]}
        return {f"lr_scheduler_{i}": s for i, s in enumerate(self.schedulers)}
