"""Training-time attention.

`attention(q, k, v, ...)` takes [batch, seq, heads, head_dim] tensors (GQA when k/v have fewer
heads) and supports causal, sliding-window, soft-capped and packed-document (varlen) masks.
`packed_qkv_attention` consumes the output of one fused QKV projection, applies RoPE in
place and returns the gradient as one packed tensor, so the projection's dgrad / wgrad
GEMMs see a single operand.

The softmax(QK^T)V core runs on PyTorch's fused scaled-dot-product kernels on CUDA (the
stand-in for a tcgen05 training attention kernel); masks that those kernels do not take are
evaluated by the eager fp32 path, which is also the CPU oracle.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

import halite_b200.ops as ops
from halite_b200.ops.rope import apply_rope_reference


def attention_reference(q, k, v, causal=True, scale=None, softcap=0.0, window=None, mask=None,
                        bias=None, document_ids=None, q_offset=0):
    """Eager fp32 attention. q: [B,Sq,Hq,D]; k, v: [B,Sk,Hk,D]. `mask` is True where attention
    is NOT allowed (broadcastable to [B,H,Sq,Sk]). `document_ids` [B,S] restricts attention to
    tokens of the same document (packed sequences)."""
    B, Sq, Hq, D = q.shape
    Sk, Hk = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3)
    vf = v.float().permute(0, 2, 1, 3)
    if Hk != Hq:
        rep = Hq // Hk
        kf = kf.repeat_interleave(rep, 1)
        vf = vf.repeat_interleave(rep, 1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if softcap and softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    if bias is not None:
        s = s + bias.float()
    neg = torch.finfo(torch.float32).min
    qi = torch.arange(Sq, device=q.device).unsqueeze(-1) + (Sk - Sq if q_offset is None else q_offset)
    ki = torch.arange(Sk, device=q.device).unsqueeze(0)
    banned = torch.zeros(Sq, Sk, dtype=torch.bool, device=q.device)
    if causal:
        banned |= ki > qi
    if window is not None:
        banned |= ki <= qi - window
    s = s.masked_fill(banned, neg)
    if document_ids is not None:
        same = document_ids[:, -Sq:].unsqueeze(-1) == document_ids.unsqueeze(-2)
        s = s.masked_fill(~same.unsqueeze(1), neg)
    if mask is not None:
        s = s.masked_fill(mask, neg)
    p = torch.softmax(s, -1)
    out = torch.matmul(p, vf)
    return out.permute(0, 2, 1, 3).to(q.dtype)


def _sdpa(q, k, v, causal, scale):
    """q,k,v: [B,S,H,D] (any strides with unit inner stride) -> [B,S,H,D]."""
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    gqa = kh.shape[1] != qh.shape[1]
    out = F.scaled_dot_product_attention(qh, kh, vh, None, 0.0, is_causal=causal, scale=scale,
                                         enable_gqa=gqa)
    return out.transpose(1, 2)


def attention(q, k, v, causal=True, scale=None, softcap=0.0, window=None, mask=None, bias=None,
              document_ids=None, cu_seqlens=None, max_seqlen=None):
    """Dispatch: fused kernels for plain causal / full attention in bf16/fp16 on CUDA; eager
    fp32 otherwise. Varlen input ([1, total, H, D] with `cu_seqlens`) is handled per document."""
    if cu_seqlens is not None:
        return varlen_attention(q, k, v, cu_seqlens, max_seqlen, causal, scale, softcap, window)
    plain = softcap in (0, 0.0, None) and window is None and mask is None and bias is None \
        and document_ids is None
    if plain and q.is_cuda and q.dtype in (torch.bfloat16, torch.float16) and not ops.force_reference():
        return _sdpa(q, k, v, causal and q.shape[1] > 1, scale)
    return attention_reference(q, k, v, causal, scale, softcap, window, mask, bias, document_ids,
                               q_offset=None)


def varlen_attention(q, k, v, cu_seqlens, max_seqlen=None, causal=True, scale=None, softcap=0.0,
                     window=None):
    """Packed sequences: q,k,v [total, H, D] (or [1,total,H,D]); cu_seqlens [n+1] int."""
    squeeze = q.dim() == 4
    if squeeze:
        q, k, v = q[0], k[0], v[0]
    bounds = cu_seqlens.tolist()
    outs = []
    for s, e in zip(bounds[:-1], bounds[1:]):
        outs.append(attention(q[None, s:e], k[None, s:e], v[None, s:e], causal, scale, softcap,
                              window)[0])
    out = torch.cat(outs, 0)
    return out[None] if squeeze else out


class _PackedQKVAttention(torch.autograd.Function):
    """qkv: [B, S, (Hq + 2 Hk) * D] -> out [B, S, Hq * D]; RoPE applied in place on q, k."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, positions, n_heads, n_kv, head_dim, interleaved, causal, scale):
        C = ops.ext()
        B, S, _ = qkv.shape
        qd, kd = n_heads * head_dim, n_kv * head_dim
        q = qkv[..., :qd].unflatten(-1, (n_heads, head_dim))
        k = qkv[..., qd:qd + kd].unflatten(-1, (n_kv, head_dim))
        v = qkv[..., qd + kd:].unflatten(-1, (n_kv, head_dim))
        pos = None
        if cos is not None:
            pos = positions.expand(B, S).reshape(-1).contiguous()
            rot = cos.shape[-1] * 2
            # q and k heads are neighbours in the packed row: one launch rotates both
            C.rope_(qkv[..., :qd + kd].unflatten(-1, (n_heads + n_kv, head_dim)), cos, sin, pos, rot,
                    interleaved, False)
        if not ctx.needs_input_grad[0]:
            return _sdpa(q, k, v, causal and S > 1, scale).reshape(B, S, qd)
        with torch.enable_grad():
            qd_, kd_, vd_ = (t.detach().requires_grad_(True) for t in (q, k, v))
            out = _sdpa(qd_, kd_, vd_, causal and S > 1, scale)
        ctx.inner = (qd_, kd_, vd_, out)
        ctx.rope = (cos, sin, pos, interleaved)
        ctx.dims = (B, S, n_heads, n_kv, head_dim)
        return out.detach().reshape(B, S, qd)

    @staticmethod
    def backward(ctx, dout):
        C = ops.ext()
        qd_, kd_, vd_, out = ctx.inner
        ctx.inner = None
        B, S, H, Hk, D = ctx.dims
        dq, dk, dv = torch.autograd.grad(out, (qd_, kd_, vd_), dout.reshape(B, S, H, D))
        dqkv = torch.empty(B, S, (H + 2 * Hk) * D, device=dout.device, dtype=dout.dtype)
        qd, kd = H * D, Hk * D
        gq = dqkv[..., :qd].unflatten(-1, (H, D))
        gk = dqkv[..., qd:qd + kd].unflatten(-1, (Hk, D))
        gv = dqkv[..., qd + kd:].unflatten(-1, (Hk, D))
        cos, sin, pos, interleaved = ctx.rope
        rot = cos.shape[-1] * 2 if cos is not None else 0
        # each gradient is read once and lands, un-rotated, in its slot of the packed gradient
        for src, dst, r in ((dq, gq, rot), (dk, gk, rot), (dv, gv, 0)):
            if src.stride(-1) != 1 or src.stride(-2) != D:
                src = src.contiguous()
            C.rope_copy(src, dst, cos if r else None, sin if r else None, pos if r else None, r, interleaved, True)
        return dqkv, None, None, None, None, None, None, None, None, None


def packed_qkv_attention(qkv, n_heads, n_kv_heads, head_dim, cos=None, sin=None, positions=None,
                         interleaved=True, causal=True, scale=None):
    """Attention over a packed QKV projection output (modified in place by RoPE)."""
    if ops.use_sm100(qkv) and qkv.is_contiguous():
        return _PackedQKVAttention.apply(qkv, cos, sin, positions, n_heads, n_kv_heads, head_dim,
                                         interleaved, causal, scale)
    B, S, _ = qkv.shape
    qd, kd = n_heads * head_dim, n_kv_heads * head_dim
    q = qkv[..., :qd].unflatten(-1, (n_heads, head_dim))
    k = qkv[..., qd:qd + kd].unflatten(-1, (n_kv_heads, head_dim))
    v = qkv[..., qd + kd:].unflatten(-1, (n_kv_heads, head_dim))
    if cos is not None:
        q = apply_rope_reference(q, cos, sin, positions, interleaved)
        k = apply_rope_reference(k, cos, sin, positions, interleaved)
    return attention(q, k, v, causal, scale).reshape(B, S, qd)
