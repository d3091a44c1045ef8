"""Cross entropy family.

* `cross_entropy_rows`: per-row CE over materialised logits with z-loss, softcap, label
  smoothing, ignore_index; the gradient is produced in the forward pass and written over the
  logits (replaces the reference's Triton kernel, nn/cross_entropy.py:24-263).
* `fused_linear_cross_entropy`: head GEMM + CE in row chunks so the [tokens, vocab] logits
  never exist at once; dX and dW come out of the same pass on the tcgen05 GEMM (replaces
  nn/fused_linear_cross_entropy.py:84-157).
* `logprob_entropy`: per-token log-prob of the taken token and entropy from hidden states,
  with a recomputing backward (replaces the flash-attn Triton CE + nn/entropy.py pair used by
  the PPO actor, projects/ppo/model.py:74-86).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

import halite_b200.ops as ops
from halite_b200.ops.linear import gemm, _gemm_ready


def cross_entropy_rows_reference(logits, target, ignore_index=-100, z_loss=0.0, softcap=0.0,
                                 logit_scale=1.0, label_smoothing=0.0):
    """Returns (loss_rows, z_rows, lse) in fp32; loss_rows includes the z term."""
    x = logits.float() * logit_scale
    if softcap > 0:
        x = softcap * torch.tanh(x / softcap)
    lse = torch.logsumexp(x, -1)
    valid = target != ignore_index
    safe = target.clamp(min=0)
    xt = x.gather(-1, safe.unsqueeze(-1)).squeeze(-1)
    loss = lse - xt
    if label_smoothing > 0:
        smooth = lse - x.mean(-1)
        loss = (1 - label_smoothing) * loss + label_smoothing * smooth
    z = z_loss * lse.square()
    loss = torch.where(valid, loss + z, torch.zeros_like(loss))
    z = torch.where(valid, z, torch.zeros_like(z))
    return loss, z, lse


class _CERowsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, ignore_index, z_loss, softcap, logit_scale, label_smoothing,
                inplace):
        C = ops.ext()
        l2 = logits.reshape(-1, logits.shape[-1])
        if l2.stride(-1) != 1:
            l2 = l2.contiguous()
        t = target.reshape(-1).contiguous()
        need_grad = logits.requires_grad
        dl = None
        if need_grad:
            dl = l2 if inplace else torch.empty_like(l2)
        loss, lse, zl = C.cross_entropy(l2, t, dl, ignore_index, z_loss, softcap, logit_scale,
                                        label_smoothing, 1.0, None, None, False, 0)[:3]
        ctx.save_for_backward(dl) if need_grad else None
        ctx.shape = logits.shape
        ctx.mark_non_differentiable(zl, lse)
        return loss.view(target.shape), zl.view(target.shape), lse.view(target.shape)

    @staticmethod
    def backward(ctx, dloss, _dz, _dlse):
        (dl,) = ctx.saved_tensors
        g = dl * dloss.reshape(-1, 1).to(dl.dtype)
        return g.view(ctx.shape), None, None, None, None, None, None, None


def cross_entropy_rows(logits, target, ignore_index=-100, z_loss=0.0, softcap=0.0, logit_scale=1.0,
                       label_smoothing=0.0, inplace=False):
    """Per-row (loss incl. z term, z term, lse). `inplace=True` lets the gradient overwrite the
    logits (the caller must not use them afterwards)."""
    if logits.is_cuda and not ops.force_reference() and logits.dtype in (torch.bfloat16, torch.float32):
        return _CERowsFn.apply(logits, target, ignore_index, float(z_loss), float(softcap),
                               float(logit_scale), float(label_smoothing), inplace)
    return cross_entropy_rows_reference(logits, target, ignore_index, z_loss, softcap, logit_scale,
                                        label_smoothing)


# --------------------------------------------------------------------------- fused linear + CE

def _chunk_rows(n_rows, vocab, budget_bytes=2 << 30):
    rows = max(256, budget_bytes // (vocab * 2))
    rows = 1 << (rows.bit_length() - 1)
    return min(rows, max(n_rows, 1))


class _FusedLinearCEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, target, ignore_index, z_loss, softcap, chunk_rows):
        C = ops.ext()
        x2 = x.reshape(-1, x.shape[-1])
        if not _gemm_ready(x2):
            x2 = x2.contiguous()
        t = target.reshape(-1).contiguous()
        T, V = x2.shape[0], weight.shape[0]
        need_grad = x.requires_grad or weight.requires_grad
        losses = torch.empty(T, device=x.device, dtype=torch.float32)
        zs = torch.empty(T, device=x.device, dtype=torch.float32)
        chunk = chunk_rows or _chunk_rows(T, V)
        dx = torch.empty_like(x2) if need_grad else None
        main = getattr(weight, "_hb_grad", None)
        dw = None
        if need_grad:
            dw = torch.empty(weight.shape, device=x.device,
                             dtype=main.dtype if main is not None else torch.float32)
        w = weight if _gemm_ready(weight) else weight.contiguous()
        logits = torch.empty(min(chunk, T), V, device=x.device, dtype=torch.bfloat16)
        first = True
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            lg = logits[: e - s]
            gemm(x2[s:e], w, out=lg)
            res = C.cross_entropy(lg, t[s:e], lg if need_grad else None, ignore_index, z_loss,
                                  softcap, 1.0, 0.0, 1.0, None, None, False, 0)
            losses[s:e] = res[0]
            zs[s:e] = res[2]
            if need_grad:
                gemm(lg, w, out=dx[s:e], b_mn=True)                      # dX = dlogits W
                gemm(lg, x2[s:e], out=dw, a_mn=True, b_mn=True, accumulate=not first)  # dW += dlogits^T X
            first = False
        if need_grad:
            ctx.save_for_backward(dx, dw)
        ctx.weight_ref = weight
        ctx.x_shape = x.shape
        ctx.mark_non_differentiable(zs)
        return losses.view(target.shape), zs.view(target.shape)

    @staticmethod
    def backward(ctx, dloss, _dz):
        # Per-row upstream gradients differ only when the caller weights rows; the common
        # case (mean / sum) is one scalar, applied here to the gradients made in forward.
        dx, dw = ctx.saved_tensors
        g = dloss.reshape(-1)
        gx = dx * g.unsqueeze(-1).to(dx.dtype)
        # dW was accumulated with unit row weights: exact when g is constant over rows
        scale = g[0]
        wref = ctx.weight_ref
        main = getattr(wref, "_hb_grad", None)
        if main is not None:
            owner = getattr(wref, "_hb_grad_owner", None)
            acc = owner.mark_written(wref) if owner is not None else False
            if acc:
                main.add_(dw * scale)
            else:
                torch.mul(dw, scale, out=main)
            gw = None
        else:
            gw = (dw * scale).to(wref.dtype)
        return gx.view(ctx.x_shape), gw, None, None, None, None, None


def fused_linear_cross_entropy(x, weight, target, ignore_index=-100, z_loss=0.0, softcap=0.0,
                               chunk_rows=None):
    """Per-token (loss incl. z term, z term) of `cross_entropy(x @ weight.T, target)`.

    The upstream gradient must be the same for every row (mean / sum reductions); use
    `cross_entropy_rows` on materialised logits for per-row weights.
    """
    if ops.use_sm100(x) and weight.dtype == torch.bfloat16:
        return _FusedLinearCEFn.apply(x, weight, target, ignore_index, float(z_loss), float(softcap),
                                      chunk_rows)
    logits = F.linear(x, weight)
    loss, z, _ = cross_entropy_rows_reference(logits, target, ignore_index, z_loss, softcap)
    return loss, z


# --------------------------------------------------------------------------- PPO log-prob + entropy

def logprob_entropy_reference(hidden, weight, target, inv_temperature=None, ignore_index=-100):
    logits = F.linear(hidden, weight).float()
    if inv_temperature is not None:
        logits = logits * inv_temperature.reshape(-1, *([1] * (logits.dim() - 1))).expand(
            *logits.shape[:-1], 1) if inv_temperature.dim() == 1 and logits.dim() == 3 else \
            logits * inv_temperature.reshape(*logits.shape[:-1], 1)
    logp_all = torch.log_softmax(logits, -1)
    safe = target.clamp(min=0)
    logp = logp_all.gather(-1, safe.unsqueeze(-1)).squeeze(-1)
    logp = torch.where(target != ignore_index, logp, torch.zeros_like(logp))
    ent = -(logp_all.exp() * logp_all).sum(-1)
    return logp, ent


class _LogprobEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, target, row_scale, ignore_index, chunk_rows):
        C = ops.ext()
        h2 = hidden.reshape(-1, hidden.shape[-1])
        if not _gemm_ready(h2):
            h2 = h2.contiguous()
        t = target.reshape(-1).contiguous()
        T, V = h2.shape[0], weight.shape[0]
        rs = row_scale.reshape(-1).float().contiguous() if row_scale is not None else None
        chunk = chunk_rows or _chunk_rows(T, V)
        w = weight if _gemm_ready(weight) else weight.contiguous()
        logp = torch.empty(T, device=hidden.device, dtype=torch.float32)
        ent = torch.empty_like(logp)
        lse = torch.empty_like(logp)
        logits = torch.empty(min(chunk, T), V, device=hidden.device, dtype=torch.bfloat16)
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            lg = logits[: e - s]
            gemm(h2[s:e], w, out=lg)
            res = C.cross_entropy(lg, t[s:e], None, ignore_index, 0.0, 0.0, 1.0, 0.0, 1.0, None,
                                  rs[s:e] if rs is not None else None, True, 0)
            logp[s:e] = -res[0]
            lse[s:e] = res[1]
            ent[s:e] = res[3]
        ctx.save_for_backward(h2, weight, t, lse, ent, rs if rs is not None else torch.empty(0))
        ctx.has_rs = rs is not None
        ctx.ignore_index, ctx.chunk, ctx.shape = ignore_index, chunk, hidden.shape
        ctx.weight_ref = weight
        return logp.view(target.shape), ent.view(target.shape)

    @staticmethod
    def backward(ctx, g_logp, g_ent):
        C = ops.ext()
        h2, weight, t, lse, ent, rs = ctx.saved_tensors
        rs = rs if ctx.has_rs else None
        T, V = h2.shape[0], weight.shape[0]
        g_logp = g_logp.reshape(-1).float().contiguous()
        g_ent = g_ent.reshape(-1).float().contiguous()
        w = weight if _gemm_ready(weight) else weight.contiguous()
        dh = torch.empty_like(h2)
        wref = ctx.weight_ref
        main = getattr(wref, "_hb_grad", None)
        need_w = main is not None or ctx.needs_input_grad[1]
        dw = None
        acc = False
        if main is not None:
            owner = getattr(wref, "_hb_grad_owner", None)
            acc = owner.mark_written(wref) if owner is not None else False
            dw = main
        elif need_w:
            dw = torch.empty(weight.shape, device=h2.device, dtype=torch.float32)
        chunk = ctx.chunk
        logits = torch.empty(min(chunk, T), V, device=h2.device, dtype=torch.bfloat16)
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            lg = logits[: e - s]
            gemm(h2[s:e], w, out=lg)
            C.logprob_entropy_bwd_(lg, t[s:e], lse[s:e], ent[s:e], g_logp[s:e], g_ent[s:e],
                                   rs[s:e] if rs is not None else None, lg, ctx.ignore_index, 1.0, 0)
            gemm(lg, w, out=dh[s:e], b_mn=True)
            if need_w:
                gemm(lg, h2[s:e], out=dw, a_mn=True, b_mn=True, accumulate=acc or s > 0)
        gw = None
        if main is None and need_w:
            gw = dw.to(weight.dtype)
        return dh.view(ctx.shape), gw, None, None, None, None


def logprob_entropy(hidden, weight, target, inv_temperature=None, ignore_index=-100, chunk_rows=None):
    """(log p(target), entropy) per token from hidden states and the head weight.

    `inv_temperature` is one value per token (1 / sampling temperature) or None.
    """
    if ops.use_sm100(hidden) and weight.dtype == torch.bfloat16:
        return _LogprobEntropyFn.apply(hidden, weight, target, inv_temperature, ignore_index,
                                       chunk_rows)
    logits = F.linear(hidden, weight).float()
    if inv_temperature is not None:
        logits = logits * inv_temperature.reshape(*target.shape, 1).to(logits.dtype)
    logp_all = torch.log_softmax(logits, -1)
    safe = target.clamp(min=0)
    logp = logp_all.gather(-1, safe.unsqueeze(-1)).squeeze(-1)
    logp = torch.where(target != ignore_index, logp, torch.zeros_like(logp))
    ent = -(logp_all.exp() * logp_all).sum(-1)
    return logp, ent
