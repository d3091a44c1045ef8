"""AdamW over the flat fp32 master shards of a sharded model.

One fused kernel per unit range reads the reduced fp32 gradient shard, applies the (deferred)
clipping coefficient from a device scalar, updates master / moments and writes the bf16
working shard in place inside the unit's gathered parameter buffer; then the per-unit
all-gathers are queued unit by unit in forward order. Nothing in `step()` synchronises with the host.

Replaces `torch.optim.AdamW(foreach)` + `clip_grad_norm_(foreach)` on DTensor shards in the
reference's loop (scripts/lm.py:94-100).
"""

from __future__ import annotations

import torch

from halite_b200 import ops
from halite_b200.parallel import comm


class ShardedAdamW(torch.optim.Optimizer):
    def __init__(self, model, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                 amsgrad=False, **unused):
        if amsgrad:
            raise ValueError("ShardedAdamW does not implement amsgrad")
        self.fsdp = model._hb_fsdp
        self.units = self.fsdp.units
        decay, no_decay = [], []
        self._slots = []   # (unit, lo, hi, group index)
        for u in self.units:
            if u.master is None:
                u.init_master()
            (d_lo, d_hi), (n_lo, n_hi) = u.decay_split()
            if d_hi > d_lo:
                decay.append(u.master[d_lo:d_hi])
                self._slots.append((u, d_lo, d_hi, 0))
            if n_hi > n_lo:
                no_decay.append(u.master[n_lo:n_hi])
                self._slots.append((u, n_lo, n_hi, 1))
        defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
        groups = [{"params": decay, "weight_decay": weight_decay},
                  {"params": no_decay, "weight_decay": 0.0}]
        groups = [g for g in groups if g["params"]] or [{"params": [torch.zeros(0)]}]
        self._group_of = {}
        super().__init__(groups, defaults)
        self._gidx = {0: 0, 1: (1 if decay and no_decay else 0)}
        dev = self.units[0].device
        self.exp_avg = {id(u): torch.zeros_like(u.master) for u in self.units}
        self.exp_avg_sq = {id(u): torch.zeros_like(u.master) for u in self.units}
        self._step = 0
        self.clip_coef = None   # device fp32 [2]: (coefficient, norm), set by clip_grad_norm_

    @property
    def step_count(self):
        return self._step

    def zero_grad(self, set_to_none=True):
        # flat gradient buffers are overwritten by the first wgrad of the next step
        for u in self.units:
            u._written.clear()
            u._backward_done = False

    @torch.no_grad()
    def step(self, closure=None):
        self.fsdp.finish_backward()
        self.fsdp.wait_reductions()
        self._step += 1
        for u in self.units:
            if u.fused is not None:
                u.fused.wait_readers()     # peers still copying last step's shard finish first
            if u.fused_reduce is not None:
                u.fused_reduce.wait_readers()   # ... and peers still summing this step's gradients
        # unit by unit in the order the next forward uses them: a unit's gather starts on the
        # communication stream as soon as its own update is done and runs under the next units'
        # updates, and the forward only ever waits for the unit it is about to use
        by_unit = {}
        for slot in self._slots:
            by_unit.setdefault(id(slot[0]), []).append(slot)
        for u in self.units:
            for _, lo, hi, gi in by_unit.get(id(u), ()):
                g = self.param_groups[self._gidx[gi]]
                ops.fused_adamw_step(
                    u.master[lo:hi], self.exp_avg[id(u)][lo:hi], self.exp_avg_sq[id(u)][lo:hi],
                    u.grad_shard[lo:hi], u.param_shard()[lo:hi], g["lr"], g["betas"], g["eps"],
                    g["weight_decay"], self._step, 1.0, self.clip_coef)
            u._written.clear()          # the next backward pass starts a new sum
            u.start_gather(epoch=self._step)
        self.clip_coef = None

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self):
        out = {"step": self._step,
               "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}
        for u in self.units:
            out[f"{u.name}.master"] = u.master
            out[f"{u.name}.exp_avg"] = self.exp_avg[id(u)]
            out[f"{u.name}.exp_avg_sq"] = self.exp_avg_sq[id(u)]
        return out

    def load_state_dict(self, state):
        self._step = int(state["step"])
        for g, saved in zip(self.param_groups, state.get("param_groups", [])):
            g.update(saved)
        for u in self.units:
            u.master.copy_(state[f"{u.name}.master"])
            self.exp_avg[id(u)].copy_(state[f"{u.name}.exp_avg"])
            self.exp_avg_sq[id(u)].copy_(state[f"{u.name}.exp_avg_sq"])
            u.param_shard().copy_(u.master)
            if u.fused is not None:
                u.fused.wait_readers()
            u.start_gather(epoch=self._step)


@torch.no_grad()
def clip_grad_norm_(model, max_norm, optimizer=None, norm_type=2.0):
    """Global gradient norm over all shards (returned as a device tensor). For a sharded model
    the scaling is deferred: the clip coefficient is handed to the optimizer, whose fused
    kernel multiplies the gradient as it reads it. For a plain model this is
    `torch.nn.utils.clip_grad_norm_`."""
    fsdp = getattr(model, "_hb_fsdp", None)
    if fsdp is None:
        return torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm, norm_type)
    fsdp.finish_backward()
    fsdp.wait_reductions()
    dev = fsdp.units[0].device
    total = torch.zeros(1, dtype=torch.float32, device=dev)
    for u in fsdp.units:
        ops.grad_sumsq(u.grad_shard, total)
    tp = getattr(model, "_hb_tp", None)
    if tp is not None and tp.size > 1:
        # parameters replicated over tensor-parallel ranks must count once, sharded ones on
        # every rank: discount the replicated part before summing over the TP group
        rep = torch.zeros(1, dtype=torch.float32, device=dev)
        for u in fsdp.units:
            for m, n, _, off, numel in u.entries:
                if getattr(m._parameters[n], "_hb_tp_replicated", None) is None:
                    continue
                a, b = max(off, u.lo) - u.lo, min(off + numel, u.hi) - u.lo
                if b > a:
                    ops.grad_sumsq(u.grad_shard[a:b], rep)
        total = total - rep * (1.0 - 1.0 / tp.size)
        comm.all_reduce(total, tp.group)
    if fsdp.shard_group is not None:
        comm.all_reduce(total, fsdp.shard_group)
    out = torch.empty(2, dtype=torch.float32, device=dev)
    if dev.type == "cuda" and not ops.force_reference():
        ops.ext().clip_coef_(total, float(max_norm or 0.0), out)
    else:
        norm = total.sqrt()
        out[0] = torch.clamp(max_norm / (norm + 1e-6), max=1.0)[0] if max_norm else 1.0
        out[1] = norm[0]
    if optimizer is not None:
        optimizer.clip_coef = out
    else:
        for u in fsdp.units:
            u.grad_shard.mul_(out[0])
    return out[1]
