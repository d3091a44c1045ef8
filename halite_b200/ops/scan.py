"""First-order recurrences over packed rows.

`linear_scan`  h[t] = a[t] * h[t-1] + b[t] * x[t]  inside every sequence of a packed row (h = 0
before a sequence's first token), forward in time or, with `reverse`, from each sequence's last
token down to its first, which is the adjoint of the forward recurrence.

`ema_scan`  h[t] = (1 - p[t]) * h[t-1] + p[t] * x[t]: the smoothing the H-Net dechunk applies to the
chunk vectors, with gradients for x and p. The reference gets it from mamba-ssm's chunked-scan
Triton kernel (transformers/models/hnet.py:88-131: A = -1, dt = log(1 / (1 - p)), B = p, C = 1);
here it is one CUDA kernel per direction (`linear_scan_kernel` in csrc/ops.cu) and a handful of
elementwise ops for the gradients (`_LinearScanFn`); with a = 1 - p and b = p they combine to

    adj[t] = g[t] + (1 - p[t+1]) * adj[t+1]          (reverse scan of the incoming gradient)
    dx[t]  = p[t] * adj[t]
    dp[t]  = sum_c adj[t, c] * (x[t, c] - h[t-1, c])

`linear_scan_autograd` is the general differentiable form; the Mamba-2 mixer uses it to pass the
state from chunk to chunk.
"""

from __future__ import annotations

import torch

from halite_b200 import ops


def _linear_scan_reference(x, a, b, cu_seqlens, reverse=False):
    """Plain PyTorch: a loop over time, vectorised over channels (CPU path and test oracle)."""
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    xf, bounds = x.float(), cu_seqlens.tolist()
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        h = torch.zeros(x.shape[1], dtype=torch.float32, device=x.device)
        steps = range(hi - 1, lo - 1, -1) if reverse else range(lo, hi)
        for t in steps:
            h = a[t] * h + b[t] * xf[t]
            out[t] = h
    return out


def linear_scan(x, a, b, cu_seqlens, reverse=False):
    """x [total, dim] (bf16 or fp32), a, b [total] fp32, cu_seqlens [n + 1] -> fp32 [total, dim]."""
    if x.is_cuda and not ops.force_reference():
        return ops.ext().linear_scan(x.contiguous(), a.float().contiguous(), b.float().contiguous(),
                                     cu_seqlens.to(device=x.device, dtype=torch.int32).contiguous(), reverse)
    return _linear_scan_reference(x, a.float(), b.float(), cu_seqlens, reverse)


class _LinearScanFn(torch.autograd.Function):
    """y[t] = a[t] y[t-1] + b[t] x[t] with gradients for x, a and b:

        adj[t] = g[t] + a[t+1] * adj[t+1]            (the same recurrence run backwards over g)
        dx[t] = b[t] * adj[t],  db[t] = sum_c adj[t, c] * x[t, c],  da[t] = sum_c adj[t, c] * y[t-1, c]
    """

    @staticmethod
    def forward(ctx, x, a, b, cu_seqlens):
        a, b = a.float(), b.float()
        y = linear_scan(x, a, b, cu_seqlens)
        ctx.save_for_backward(x, a, b, y, cu_seqlens)
        return y

    @staticmethod
    def backward(ctx, g):
        x, a, b, y, cu = ctx.saved_tensors
        total = x.shape[0]
        carry = torch.roll(a, -1)                          # carry[t] = a[t+1]; unused at a sequence's end
        adj = linear_scan(g.contiguous(), carry, torch.ones_like(a), cu, reverse=True)
        dx = (b[:, None] * adj).to(x.dtype) if ctx.needs_input_grad[0] else None
        da = db = None
        if ctx.needs_input_grad[1]:
            # y[t-1], with zeros where a sequence starts (one spare row takes the start marker of an
            # empty trailing sequence)
            y_prev = y.new_zeros(total + 1, y.shape[1])
            y_prev[1:total] = y[: total - 1]
            y_prev.index_fill_(0, cu[:-1].to(device=y.device, dtype=torch.long), 0.0)
            da = (adj * y_prev[:total]).sum(-1)
        if ctx.needs_input_grad[2]:
            db = (adj * x.float()).sum(-1)
        return dx, da, db, None


def linear_scan_autograd(x, a, b, cu_seqlens):
    """Differentiable `linear_scan` (forward direction): x [total, dim], a, b [total] -> fp32 [total, dim]."""
    return _LinearScanFn.apply(x, a, b, cu_seqlens)


def ema_scan(x, p, cu_seqlens):
    """h[t] = (1 - p[t]) h[t-1] + p[t] x[t] per sequence: x [total, dim], p [total] -> fp32 [total, dim]."""
    p = p.float()
    return _LinearScanFn.apply(x, 1 - p, p, cu_seqlens)
