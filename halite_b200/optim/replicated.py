"""Any `torch.optim` optimizer on a model wrapped for replicated data parallelism.

With `parallelize(..., data_parallel="ddp")` the model keeps the flat-buffer layout of the
sharding layer with a shard group of one rank: every rank holds whole parameters (low
precision, views of a unit's `full_param`) and, after the gradient all-reduce, whole fp32
gradients (views of `full_grad`). Optimizers that need whole weight matrices (SOAP, Shampoo;
reference: configs/lm/scale_383m_shampoo.py:75-90, optim/soap.py) run here on fp32 master
copies:

    master[p]  fp32 nn.Parameter, a view of the unit's fp32 master buffer
    .grad      the matching view of the unit's reduced fp32 gradient (scaled by the clip
               coefficient that `clip_grad_norm_` leaves on the optimizer)
    step()     inner.step() on the masters, then one cast of each master buffer back into
               the low-precision parameters the model computes with
"""

from __future__ import annotations

import torch
from torch import nn


class ReplicatedOptimizer:
    def __init__(self, model, factory, weight_decay: float = 0.0):
        self._sharding = model._hb_fsdp      # (not named `fsdp`: checkpointing treats this as a plain optimizer)
        self.units = self._sharding.units
        if any(u.ws != 1 for u in self.units):
            raise TypeError("this optimizer needs whole parameters: wrap the model with data_parallel='ddp'")
        decay, no_decay = [], []
        self._views = []        # (master parameter, unit, offset, numel)
        for u in self.units:
            if u.master is None:
                u.init_master()
            for m, n, _, off, numel in u.entries:
                p = m._parameters[n]
                if not p.requires_grad:
                    continue
                mp = nn.Parameter(u.master[off:off + numel].view(p.shape))
                self._views.append((mp, u, off, numel))
                (no_decay if p.ndim < 2 else decay).append(mp)
        groups = [g for g in ({"params": decay, "weight_decay": weight_decay},
                              {"params": no_decay, "weight_decay": 0.0}) if g["params"]]
        self.inner = factory(groups)
        self.clip_coef = None   # device fp32 [2]: (coefficient, norm), set by clip_grad_norm_
        self._step = 0

    # what schedulers, loggers and checkpoints touch
    @property
    def param_groups(self):
        return self.inner.param_groups

    @property
    def state(self):
        return self.inner.state

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
        self._sharding.finish_backward()
        self._sharding.wait_reductions()
        self._step += 1
        coef = None if self.clip_coef is None else self.clip_coef[0]
        for mp, u, off, numel in self._views:
            g = u.grad_shard[off:off + numel].view(mp.shape)
            if g.dtype != torch.float32:
                g = g.float()
            mp.grad = g * coef if coef is not None else g
        self.clip_coef = None
        self.inner.step()
        for u in self.units:
            u.param_shard().copy_(u.master)
            u._written.clear()          # the next backward pass starts a new sum
            u.start_gather(epoch=self._step)

    def state_dict(self):
        """The inner optimizer's state dict (torch layout: `state` by parameter index, `param_groups`),
        with each parameter's fp32 master stored beside its state and the step count beside the first."""
        sd = self.inner.state_dict()
        for pid, (mp, _, _, _) in enumerate(self._views):
            sd["state"].setdefault(pid, {})["master"] = mp.detach()
        sd["state"].setdefault(0, {})["replicated_step"] = torch.tensor(self._step)
        return sd

    def load_state_dict(self, state):
        state = {"state": {k: dict(v) for k, v in state["state"].items()}, "param_groups": state["param_groups"]}
        step = state["state"].get(0, {}).pop("replicated_step", None)
        if step is not None:
            self._step = int(step)
        with torch.no_grad():
            for pid, (mp, _, _, _) in enumerate(self._views):
                master = state["state"].get(pid, {}).pop("master", None)
                if master is not None:
                    mp.copy_(master)
        state["state"] = {k: v for k, v in state["state"].items() if v}
        self.inner.load_state_dict(state)
        for u in self.units:
            u.param_shard().copy_(u.master)
