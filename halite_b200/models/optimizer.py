"""Post-step weight re-normalisation for nGPT (reference: transformers/optimizer.py:6-35): every
matrix is projected back onto the unit hypersphere along its embedding dimension after each
optimizer step."""

from __future__ import annotations

import torch


def calc_norm(x):
    return x.pow(2).sum(-2, keepdim=True).sqrt()


def normalize(x, dim=-1):
    return (x.float() / x.float().norm(p=2, dim=dim, keepdim=True)).to(x.dtype)


@torch.no_grad()
def ngpt_normalize(model, transposed=("out.weight",)):
    """Rows are unit-normalised, except for matrices whose name contains one of `transposed`
    (projections back into the residual stream), which are normalised along dim 0. On a sharded
    model the master copies are refreshed from the re-normalised parameters."""
    for name, p in model.named_parameters():
        if p.ndim < 2:
            continue
        dim = 0 if any(t in name for t in transposed) else 1
        p.copy_(normalize(p, dim))
    fsdp = getattr(model, "_hb_fsdp", None)
    if fsdp is not None:
        for u in fsdp.units:
            if u.master is not None:
                u.master.copy_(u.param_shard())
