"""Linear layers on the tcgen05 GEMM: forward, dgrad and wgrad with no transposes.

`linear(x, w, b)` is the replacement for every `nn.Linear.__call__` of the reference
(cuBLAS behind configs/models/transformer.py:124-177,292). On CPU / fp32 it is `F.linear`.

Main-grad protocol: when the weight tensor carries `_hb_grad` (a view into a flat gradient
buffer owned by the FSDP layer), the wgrad GEMM writes (or accumulates) straight into that
buffer in the buffer's dtype and autograd receives no weight gradient. That removes the
bf16 wgrad tensor, its cast to fp32 and the copy into the reduce-scatter buffer.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

import halite_b200.ops as ops
from halite_b200.utils import probe as _probe

_noted = set()


def _note_library_path(kind, shape):
    """Log, once per (kind, shape), that a bf16 CUDA product left the tcgen05 kernel for a library
    routine because a dimension is not a multiple of 8 (16-byte rows are what TMA needs)."""
    key = (kind, tuple(shape))
    if key in _noted:
        return
    _noted.add(key)
    from halite_b200.logging import logger

    logger.warning(f"{kind}: shape {tuple(shape)} has a dimension that is not a multiple of 8; "
                   "this product runs on the library GEMM, not on the sm_100a kernel")


def gemm(a, b, out=None, a_mn=False, b_mn=False, accumulate=False, out_dtype=None, block_n=0,
         max_ctas=0, gather=None, scatter=None, group=None):
    """out[M,N] (+)= op(a) @ op(b)^T on the sm_100a kernel.

    a: [M,K] (or [K,M] when a_mn); b: [N,K] (or [K,N] when b_mn); all bf16, row-major with
    16-byte aligned rows.
    """
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        out = torch.empty(M, N, device=a.device, dtype=out_dtype or torch.bfloat16)
    if gather is None and scatter is None and group is None and not (_tma_ready(a) and _tma_ready(b)):
        # rows that are not 16-byte multiples (a vocabulary of 260, say): the library computes it
        if a.is_cuda:
            _note_library_path("gemm", (M, N))
        prod = torch.matmul((a.t() if a_mn else a).float(), (b if b_mn else b.t()).float())
        if accumulate:
            out += prod.to(out.dtype)
        else:
            out.copy_(prod)
        return out
    ops.ext().gemm(a, b, out, a_mn, b_mn, accumulate, block_n, max_ctas, ops.status_word(a.device),
                   gather, scatter, group)
    return out


def _tma_ready(t):
    """What a TMA descriptor over a 2-D operand needs: unit inner stride, 16-byte base and rows."""
    return t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


def _as_2d(x):
    return x.reshape(-1, x.shape[-1])


def _gemm_ready(t):
    """Row-major 2-D with unit inner stride and 16-byte aligned rows / base."""
    return (t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0
            and t.data_ptr() % 16 == 0)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = _as_2d(x)
        if not _gemm_ready(x2):
            x2 = x2.contiguous()
        w = weight if _gemm_ready(weight) else weight.contiguous()
        # a data-parallel wrapper may hang another unit's parameter gather on this launch
        carry = getattr(weight, "_hb_carry", None)
        out = gemm(x2, w, gather=carry() if carry is not None else None)
        if bias is not None:
            out += bias
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        ctx.weight_ref = weight
        return out.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = _as_2d(dy)
        if not _gemm_ready(dy2):
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            # dX[M,K] = dY[M,N] @ W[N,K]: B operand is W read "MN-major"
            w = weight if _gemm_ready(weight) else weight.contiguous()
            # the gradient reduction of the unit whose backward just ended may ride on this launch
            carry = getattr(ctx.weight_ref, "_hb_carry_bwd", None)
            dx = gemm(dy2, w, b_mn=True, gather=carry() if carry is not None else None).view(ctx.x_shape)
        wref = ctx.weight_ref
        main = getattr(wref, "_hb_grad", None)
        if main is not None:
            # dW[N,K] = dY^T X accumulated in the flat gradient buffer
            owner = getattr(wref, "_hb_grad_owner", None)
            acc = owner.mark_written(wref) if owner is not None else False
            gemm(dy2, x2, out=main, a_mn=True, b_mn=True, accumulate=acc)
        elif ctx.needs_input_grad[1]:
            dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0)
        return dx, dw, db


def linear(x, weight, bias=None):
    # the kernel wants 16-byte rows in every layout it reads the operands in (forward, dgrad, wgrad):
    # both weight dimensions must be multiples of 8, otherwise the library path runs
    if ops.use_sm100(x) and weight.dtype == torch.bfloat16 and weight.shape[0] % 8 == 0 \
            and weight.shape[1] % 8 == 0 and x.dtype == torch.bfloat16:
        out = _LinearFn.apply(x, weight, bias)
    else:
        if x.is_cuda and x.dtype == torch.bfloat16 and not ops.force_reference():
            _note_library_path("linear", weight.shape)
        out = F.linear(x, weight, bias)
    if _probe.active_probe() is not None:
        _probe.active_probe().on_linear(x, weight, out)
    return out


def matmul_nt(a, b, out_dtype=None):
    """a[M,K] @ b[N,K]^T without autograd (inference paths)."""
    if ops.use_sm100(a) and b.dtype == torch.bfloat16:
        a2 = a if _gemm_ready(a) else a.contiguous()
        b2 = b if _gemm_ready(b) else b.contiguous()
        return gemm(a2, b2, out_dtype=out_dtype)
    out = a.float() @ b.float().t()
    return out.to(out_dtype or a.dtype)
