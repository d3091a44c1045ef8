"""Shampoo with Adam grafting (Gupta et al., "Shampoo: Preconditioned Stochastic Tensor
Optimization"; Anil et al., "Scalable Second Order Optimization for Deep Learning").

The reference trains one of its scaling configs with the external `distributed_shampoo` package
(configs/lm/scale_383m_shampoo.py:75-90: betas, epsilon, max_preconditioner_dim,
precondition_frequency, use_decoupled_weight_decay, inv_root_override, AdamGraftingConfig).
This is an in-tree optimizer with the same hyperparameter surface, so that config needs no
outside package.

For a gradient G of a tensor with modes d_1 .. d_k (modes larger than `max_preconditioner_dim`
are left unpreconditioned; higher-rank tensors may be folded with `merge_dims`):

    L_i <- beta2 L_i + (1 - beta2) G_(i) G_(i)^T            one factor per mode
    P_i  = (L_i + epsilon I)^(-1/root)                      refreshed every `precondition_frequency` steps
                                                            (eigenvalues floored at 1e-6 of the largest)
    S    = G x_1 P_1 x_2 ... x_k P_k                        the Shampoo direction of the filtered gradient
    U    = S * |A| / |S|                                    grafting: the step length of Adam's update A

`root` is `inv_root_override` when given, else 2k (the classic exponent -1/(2k) per factor).
Until the first refresh (`start_preconditioning_step`) the update is the grafted Adam step itself.
Works on full (unsharded) parameters: with the sharding layer use `data_parallel="ddp"`.
"""

from __future__ import annotations

import torch
from torch import optim

from .soap import _merge_dims


class AdamGraftingConfig:
    """Second-moment decay and epsilon of the Adam update whose per-tensor norm the step takes."""

    def __init__(self, beta2: float = 0.999, epsilon: float = 1e-8):
        self.beta2 = beta2
        self.epsilon = epsilon


def _inverse_root(mat, root, epsilon, floor=1e-6):
    """(mat + epsilon I)^(-1/root) of a symmetric PSD matrix through its eigendecomposition.
    Eigenvalues below `floor` x the largest one are raised to it first: the factor is accumulated
    in fp32, so anything smaller is rounding noise that a negative power would blow up."""
    n = mat.shape[0]
    sym = (mat + mat.t()) * 0.5
    try:
        vals, vecs = torch.linalg.eigh(sym.double())
    except RuntimeError:
        # a factor that lost definiteness numerically: fall back to its diagonal
        return torch.diag(torch.diagonal(sym).clamp_min(0).add(epsilon).pow(-1.0 / root)).float()
    vals = vals.clamp_min(vals.max().clamp_min(0) * floor) + epsilon
    return ((vecs * vals.pow(-1.0 / root)) @ vecs.t()).to(mat.dtype).view(n, n)


class Shampoo(optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), epsilon=1e-12, weight_decay=0.0,
                 max_preconditioner_dim=8192, precondition_frequency=10, start_preconditioning_step=None,
                 use_decoupled_weight_decay=True, inv_root_override=0, grafting_config=None, merge_dims=False,
                 precondition_1d=False, eigenvalue_floor=1e-6, distributed_config=None):
        if grafting_config is None:
            grafting_config = AdamGraftingConfig(beta2=betas[1])
        defaults = dict(lr=lr, betas=betas, epsilon=epsilon, weight_decay=weight_decay,
                        max_preconditioner_dim=max_preconditioner_dim,
                        precondition_frequency=precondition_frequency,
                        start_preconditioning_step=start_preconditioning_step or precondition_frequency,
                        use_decoupled_weight_decay=use_decoupled_weight_decay, inv_root_override=inv_root_override,
                        graft_beta2=grafting_config.beta2, graft_eps=grafting_config.epsilon,
                        merge_dims=merge_dims, precondition_1d=precondition_1d, eigenvalue_floor=eigenvalue_floor)
        super().__init__(params, defaults)

    def _init_state(self, p, g, group):
        st = self.state[p]
        st["step"] = 0
        st["exp_avg"] = torch.zeros_like(g, dtype=torch.float32)          # filtered gradient
        st["graft_sq"] = torch.zeros_like(g, dtype=torch.float32)         # Adam's second moment
        limit = group["max_preconditioner_dim"]
        skip = g.dim() == 0 or (g.dim() == 1 and not group["precondition_1d"])
        st["factors"] = [None if skip or d > limit or d == 1 else
                         torch.zeros(d, d, device=g.device, dtype=torch.float32) for d in g.shape]
        st["roots"] = [None] * len(st["factors"])
        return st

    @staticmethod
    def _precondition(g, roots):
        out = g
        for i, r in enumerate(roots):
            if r is None:
                continue
            out = torch.movedim(torch.tensordot(r, out, dims=([1], [i])), 0, i)
        return out

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad.float()
                shape = g.shape
                if group["merge_dims"] and g.dim() > 2:
                    g = g.reshape(_merge_dims(shape, group["max_preconditioner_dim"]))
                st = self.state[p] if len(self.state[p]) else self._init_state(p, g, group)
                st["step"] += 1
                step = st["step"]
                if group["weight_decay"] and not group["use_decoupled_weight_decay"]:
                    g = g + group["weight_decay"] * p.float().reshape(g.shape)

                # statistics of both halves
                for i, f in enumerate(st["factors"]):
                    if f is None:
                        continue
                    dims = [j for j in range(g.dim()) if j != i]
                    f.lerp_(torch.tensordot(g, g, dims=(dims, dims)), 1 - beta2)
                st["graft_sq"].lerp_(g * g, 1 - group["graft_beta2"])
                st["exp_avg"].lerp_(g, 1 - beta1)
                m_hat = st["exp_avg"] / (1 - beta1 ** step)
                adam = m_hat / ((st["graft_sq"] / (1 - group["graft_beta2"] ** step)).sqrt() + group["graft_eps"])

                # inverse roots, every `precondition_frequency` steps once preconditioning has started
                active = [f for f in st["factors"] if f is not None]
                if active and step >= group["start_preconditioning_step"] and \
                        (step == group["start_preconditioning_step"] or step % group["precondition_frequency"] == 0):
                    root = group["inv_root_override"] or 2 * len(active)
                    corr = 1 - beta2 ** step
                    st["roots"] = [None if f is None else _inverse_root(f / corr, root, group["epsilon"],
                                                                           group["eigenvalue_floor"])
                                   for f in st["factors"]]

                if any(r is not None for r in st["roots"]):
                    direction = self._precondition(m_hat, st["roots"])
                    update = direction * (adam.norm() / direction.norm().clamp_min(1e-30))
                else:
                    update = adam

                if group["weight_decay"] and group["use_decoupled_weight_decay"]:
                    p.mul_(1 - group["lr"] * group["weight_decay"])
                p.add_(update.reshape(shape).to(p.dtype), alpha=-group["lr"])
        return loss
