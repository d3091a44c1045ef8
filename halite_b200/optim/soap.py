"""SOAP: Adam run in the eigenbasis of Shampoo's Kronecker-factored preconditioner
(reference: optim/soap.py:11-420; algorithm of Vyas et al., "SOAP: Improving and Stabilizing
Shampoo using Adam").

For a matrix gradient G: L <- beta L + (1-beta) G G^T, R <- beta R + (1-beta) G^T G. Every
`precondition_frequency` steps the eigenvector estimates Q_L, Q_R are refreshed with one step of
power iteration + QR (a full `eigh` on first use). Adam's moments live in the rotated space
G' = Q_L^T G Q_R; the first moment is kept in the original space and rotated on use, the second
is carried across a basis refresh by rotating it with the old->new change of basis.

Works on full (unsharded) parameters: with the sharding layer use `data_parallel="ddp"`.
"""

from __future__ import annotations

import torch
from torch import optim


def _merge_dims(shape, max_dim):
    """Greedily fold trailing dimensions together while the product stays <= max_dim."""
    out, cur = [], 1
    for d in reversed(shape):
        if cur * d > max_dim:
            if cur > 1:
                out.append(cur)
            cur = d
        else:
            cur *= d
    out.append(cur)
    return tuple(reversed(out))


class _Basis:
    """Per-parameter factors `GG[i]` and eigenbases `Q[i]`, one per tensor mode (None = mode
    left unrotated because it is too large or 1-D preconditioning is off)."""

    def __init__(self, grad, max_precond_dim, precondition_1d):
        self.GG, self.Q = [], None
        if grad.dim() == 1 and (not precondition_1d or grad.shape[0] > max_precond_dim):
            self.GG = [None]
        else:
            for d in grad.shape:
                self.GG.append(None if d > max_precond_dim else
                               torch.zeros(d, d, device=grad.device, dtype=torch.float32))

    def accumulate(self, grad, beta):
        g = grad.float()
        for i, m in enumerate(self.GG):
            if m is None:
                continue
            dims = [j for j in range(g.dim()) if j != i]
            m.lerp_(torch.tensordot(g, g, dims=(dims, dims)), 1 - beta)

    def rotate(self, t, back=False):
        """Apply Q_i^T (or Q_i when `back`) along every rotated mode."""
        if self.Q is None:
            return t
        out = t.float()
        for i, q in enumerate(self.Q):
            if q is None:
                continue
            mat = q if not back else q.t()
            out = torch.movedim(torch.tensordot(out, mat, dims=([i], [0])), -1, i)
        return out.to(t.dtype)

    def init_eigh(self):
        self.Q = []
        for m in self.GG:
            if m is None:
                self.Q.append(None)
                continue
            _, vecs = torch.linalg.eigh(m + 1e-30 * torch.eye(m.shape[0], device=m.device))
            self.Q.append(vecs.flip(1).contiguous())          # descending eigenvalues

    def refresh(self, exp_avg_sq):
        """One power-iteration + QR step per mode; returns `exp_avg_sq` expressed in the new
        basis (modes re-sorted by the estimated eigenvalues so entries keep their meaning)."""
        sq = exp_avg_sq.float()
        for i, (m, q) in enumerate(zip(self.GG, self.Q)):
            if m is None:
                continue
            est = torch.einsum("ij,ij->j", q, m @ q)            # diag(Q^T GG Q)
            order = torch.argsort(est, descending=True)
            sq = sq.index_select(i, order)
            new_q, _ = torch.linalg.qr(m @ q[:, order])
            self.Q[i] = new_q
        return sq.to(exp_avg_sq.dtype)


class SOAP(optim.Optimizer):
    def __init__(self, params, lr=3e-3, betas=(0.95, 0.95), shampoo_beta=-1, eps=1e-8, weight_decay=0.01,
                 precondition_frequency=10, max_precond_dim=10000, merge_dims=False, precondition_1d=False,
                 normalize_grads=False, data_format="channels_first", correct_bias=True):
        defaults = dict(lr=lr, betas=betas, shampoo_beta=shampoo_beta, eps=eps, weight_decay=weight_decay,
                        precondition_frequency=precondition_frequency, max_precond_dim=max_precond_dim,
                        merge_dims=merge_dims, precondition_1d=precondition_1d, normalize_grads=normalize_grads,
                        correct_bias=correct_bias)
        super().__init__(params, defaults)
        self._data_format = data_format

    def _view(self, t, group):
        """The shape the preconditioner sees (optionally with small dimensions merged)."""
        if not group["merge_dims"] or t.dim() < 2:
            return t
        if t.dim() == 4 and self._data_format == "channels_last":
            t = t.permute(0, 3, 1, 2)
        return t.reshape(_merge_dims(t.shape, group["max_precond_dim"]))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            sbeta = group["shampoo_beta"] if group["shampoo_beta"] >= 0 else beta2
            for p in group["params"]:
                if p.grad is None:
                    continue
                grad = p.grad
                state = self.state[p]
                gview = self._view(grad, group)
                if "basis" not in state:
                    state["step"] = 0
                    state["exp_avg"] = torch.zeros_like(grad)
                    state["exp_avg_sq"] = torch.zeros_like(gview)
                    basis = state["basis"] = _Basis(gview, group["max_precond_dim"], group["precondition_1d"])
                    basis.accumulate(gview, sbeta)
                    basis.init_eigh()
                    continue        # the first gradient only seeds the preconditioner
                basis = state["basis"]
                state["step"] += 1
                exp_avg, exp_avg_sq = state["exp_avg"], state["exp_avg_sq"]
                g_rot = basis.rotate(gview)
                exp_avg.lerp_(grad, 1 - beta1)
                exp_avg_sq.mul_(beta2).addcmul_(g_rot, g_rot, value=1 - beta2)
                m_rot = basis.rotate(self._view(exp_avg, group))
                update = basis.rotate(m_rot / (exp_avg_sq.sqrt() + group["eps"]), back=True).reshape(grad.shape)
                step_size = group["lr"]
                if group["correct_bias"]:
                    step_size *= (1 - beta2 ** state["step"]) ** 0.5 / (1 - beta1 ** state["step"])
                if group["normalize_grads"]:
                    update = update / (1e-30 + update.square().mean().sqrt())
                p.add_(update.to(p.dtype), alpha=-step_size)
                if group["weight_decay"] > 0:
                    p.mul_(1 - group["lr"] * group["weight_decay"])
                # the current gradient enters the preconditioner only after it has been used
                basis.accumulate(gview, sbeta)
                if state["step"] % group["precondition_frequency"] == 0:
                    state["exp_avg_sq"] = basis.refresh(exp_avg_sq)
        return loss
