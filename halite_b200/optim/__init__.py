"""Optimisation helpers (reference: optim/__init__.py:4-20)."""

from __future__ import annotations


def group_parameters(model, weight_decay: float = 0.0):
    """Two parameter groups: tensors with fewer than 2 dimensions (norm scales, biases) get no
    weight decay. A model wrapped by the sharding layer is returned as a marker object that
    `build_optimizer` turns into the sharded fused optimizer."""
    fsdp = getattr(model, "_hb_fsdp", None)
    if fsdp is not None:
        return ShardedParams(model, weight_decay)
    decay, no_decay = [], []
    for p in model.parameters():
        if not p.requires_grad:
            continue
        (no_decay if p.ndim < 2 else decay).append(p)
    return [
        {"params": decay, "weight_decay": weight_decay},
        {"params": no_decay, "weight_decay": 0.0},
    ]


class ShardedParams(list):
    """What `group_parameters` returns for a sharded model; also a plain list of param groups
    so third-party optimizers still receive something sensible."""

    def __init__(self, model, weight_decay):
        self.model = model
        self.weight_decay = weight_decay
        decay = [p for p in model.parameters() if p.requires_grad and p.ndim >= 2]
        no_decay = [p for p in model.parameters() if p.requires_grad and p.ndim < 2]
        super().__init__([{"params": decay, "weight_decay": weight_decay},
                          {"params": no_decay, "weight_decay": 0.0}])


def build_optimizer(factory, model, weight_decay: float = 0.0):
    """`factory` is what a config holds (`partial(optim.AdamW, lr=..., betas=...)`). On a sharded
    model an AdamW request becomes `ShardedAdamW` (fused kernel on fp32 master shards); any other
    optimizer runs through `ReplicatedOptimizer` when the model is wrapped with
    `data_parallel="ddp"` (whole parameters on every rank)."""
    import functools

    import torch

    from .sharded_adamw import ShardedAdamW

    params = group_parameters(model, weight_decay)
    if isinstance(params, ShardedParams):
        fn = factory.func if isinstance(factory, functools.partial) else factory
        kw = dict(factory.keywords) if isinstance(factory, functools.partial) else {}
        if fn in (torch.optim.AdamW, torch.optim.Adam, ShardedAdamW):
            kw.pop("fused", None)
            kw.pop("foreach", None)
            if "weight_decay" in kw:      # the factory's own value wins only when none was passed
                wd = kw.pop("weight_decay")
                weight_decay = weight_decay if weight_decay else wd
            if fn is torch.optim.Adam:
                weight_decay = 0.0
            return ShardedAdamW(model, weight_decay=weight_decay, **kw)
        if all(u.ws == 1 for u in model._hb_fsdp.units):
            # replicated data parallelism: whole parameters on every rank, any optimizer on fp32 masters
            from .replicated import ReplicatedOptimizer

            return ReplicatedOptimizer(model, factory, weight_decay)
        raise TypeError(f"{fn} cannot drive a sharded model: it needs whole parameters. Use AdamW, or wrap the "
                        "model with data_parallel='ddp'")
    return factory(params)


from .soap import SOAP  # noqa: E402
from .lr_scheduler import PhaseScheduler, cycle_scheduler, exp_scheduler, lr_finder, step_scheduler  # noqa: E402
from .sharded_adamw import ShardedAdamW  # noqa: E402
