"""Fused optimizer pieces for flat parameter shards (one launch per shard, no host sync)."""

from __future__ import annotations

import torch

import halite_b200.ops as ops


def grad_sumsq(flat_grad: torch.Tensor, out: torch.Tensor):
    """out[0] += sum(flat_grad ** 2) in fp32."""
    if flat_grad.is_cuda and not ops.force_reference():
        ops.ext().sumsq_(flat_grad, out)
    else:
        out[0] += flat_grad.float().square().sum()
    return out


def fused_adamw_step(master, exp_avg, exp_avg_sq, grad, param_lowp, lr, betas, eps, weight_decay,
                     step, grad_scale=1.0, grad_scale_t=None):
    """Decoupled-weight-decay Adam on an fp32 master shard; `param_lowp` (bf16 copy) is
    refreshed in the same pass. Order of operations matches `torch.optim.AdamW`."""
    if master.is_cuda and not ops.force_reference():
        # the kernel refreshes a bf16 copy; parameters kept in another dtype are copied afterwards
        lowp = param_lowp if param_lowp is not None and param_lowp.dtype == torch.bfloat16 else None
        ops.ext().adamw_(master, exp_avg, exp_avg_sq, grad, lowp, lr, betas[0], betas[1], eps,
                         weight_decay, step, grad_scale, grad_scale_t)
        if param_lowp is not None and lowp is None:
            param_lowp.copy_(master)
        return
    g = grad.float() * grad_scale
    if grad_scale_t is not None:
        g = g * grad_scale_t.reshape(-1)[0]
    master.mul_(1 - lr * weight_decay)
    exp_avg.mul_(betas[0]).add_(g, alpha=1 - betas[0])
    exp_avg_sq.mul_(betas[1]).addcmul_(g, g, value=1 - betas[1])
    bc1 = 1 - betas[0] ** step
    bc2 = (1 - betas[1] ** step) ** 0.5
    denom = exp_avg_sq.sqrt() / bc2 + eps
    master.addcdiv_(exp_avg, denom, value=-lr / bc1)
    if param_lowp is not None:
        param_lowp.copy_(master)
