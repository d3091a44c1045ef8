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
    (projections back into the residual stream), which are normalised along dim 0.

    On a sharded model the projection is done on the fp32 master shards, which are the source of
    truth there (the reference normalises fp32 parameters): each rank adds up the squares of the
    master elements it owns per row (or column), the partial sums are all-reduced over the shard
    group, the rank scales its own elements, casts them into the low-precision parameters and the
    units are gathered again. Parameters are only touched after every gather in flight has landed."""
    fsdp = getattr(model, "_hb_fsdp", None)
    if fsdp is None or any(u.master is None for u in fsdp.units):
        if fsdp is not None:
            fsdp.wait_parameters()
        for name, p in model.named_parameters():
            if p.ndim < 2:
                continue
            dim = 0 if any(t in name for t in transposed) else 1
            p.copy_(normalize(p, dim))
        return
    import torch.distributed as dist

    fsdp.wait_parameters()
    names = {id(p): n for n, p in model.named_parameters()}
    for u in fsdp.units:
        jobs, sizes = [], []
        for m, n, _, off, numel in u.entries:
            p = m._parameters[n]
            if p.ndim < 2:
                continue
            rows, cols = p.shape[0], p.numel() // p.shape[0]
            along_rows = not any(t in names.get(id(p), n) for t in transposed)     # dim 1: one norm per row
            lo, hi = max(off, u.lo), min(off + numel, u.hi)
            jobs.append((off, lo, hi, cols, along_rows, rows if along_rows else cols))
            sizes.append(rows if along_rows else cols)
        if not jobs:
            continue
        sumsq = torch.zeros(sum(sizes), dtype=torch.float32, device=u.master.device)
        keys = []
        at = 0
        for off, lo, hi, cols, along_rows, n_norms in jobs:
            if hi > lo:
                idx = torch.arange(lo - off, hi - off, device=sumsq.device)
                key = (idx // cols if along_rows else idx % cols) + at
                sumsq.index_add_(0, key, u.master[lo - u.lo:hi - u.lo].square())
                keys.append(key)
            else:
                keys.append(None)
            at += n_norms
        if u.ws > 1:
            dist.all_reduce(sumsq, group=u.shard_group)
        inv = sumsq.rsqrt()
        for (off, lo, hi, cols, along_rows, n_norms), key in zip(jobs, keys):
            if key is not None:
                u.master[lo - u.lo:hi - u.lo].mul_(inv[key])
        u.param_shard().copy_(u.master)
        u.start_gather()
