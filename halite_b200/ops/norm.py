"""RMSNorm with optional fused residual add (forward and backward).

sm_100a path: `rmsnorm_fwd` / `rmsnorm_bwd` kernels (row-per-CTA forward storing rstd;
persistent-CTA backward with per-CTA weight-gradient partials). Reference semantics follow
the eager RMSNorm of the reference (nn/normalization.py:47-57): fp32 statistics, the
normalised value is cast to the input dtype before the weight multiply.
"""

from __future__ import annotations

import torch

import halite_b200.ops as ops


def rms_norm_reference(x, weight, eps, residual=None, weight_offset=0.0):
    h = x if residual is None else x + residual
    hf = h.float()
    normed = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)).type_as(h)
    out = normed if weight is None else (weight + weight_offset if weight_offset else weight) * normed
    if residual is None:
        return out
    return out, h


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, eps, weight_offset):
        C = ops.ext()
        xc = x.contiguous()
        rc = residual.contiguous() if residual is not None else None
        y, h, rstd = C.rmsnorm_fwd(xc, rc, weight, eps, weight_offset, True)
        ctx.save_for_backward(h if h is not None else xc, weight, rstd)
        ctx.has_res = residual is not None
        ctx.weight_offset = weight_offset
        if residual is not None:
            return y, h
        return y

    @staticmethod
    def backward(ctx, dy, dh=None):
        h, weight, rstd = ctx.saved_tensors
        C = ops.ext()
        dres = dh.contiguous() if (ctx.has_res and dh is not None) else None
        dx, dw = C.rmsnorm_bwd(dy.contiguous(), h, weight, rstd, dres, ctx.weight_offset)
        dw = dw.to(weight.dtype)
        if ctx.has_res:
            return dx, dx, dw, None, None
        return dx, None, dw, None, None


def rms_norm(x, weight, eps=1e-6, residual=None, weight_offset=0.0):
    """y = rmsnorm(x [+ residual]) * (weight + weight_offset).

    With `residual`, returns `(y, x + residual)` so the caller carries the summed stream on.
    """
    if weight is not None and ops.use_sm100(x) and weight.dtype == torch.bfloat16 \
            and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        return _RMSNormFn.apply(x, residual, weight, eps, weight_offset)
    return rms_norm_reference(x, weight, eps, residual, weight_offset)
