"""Training-time attention.

`attention(q, k, v, ...)` takes [batch, seq, heads, head_dim] tensors (GQA when k/v have fewer
heads) and supports causal, sliding-window, soft-capped and packed-document (varlen) masks.
`packed_qkv_attention` consumes the output of one fused QKV projection, applies RoPE in
place and returns the gradient as one packed tensor, so the projection's dgrad / wgrad
GEMMs see a single operand.

On a CUDA device in bf16 the softmax(QK^T)V core, forward and backward, is the tcgen05 kernel
pair of `csrc/attention_sm100.cu`. Every mask it takes is described by per-token segment bounds
that are built on the device (`segment_bounds_*`): a fixed batch, `cu_seqlens` packing and
per-row document offsets are the same thing to the kernel, and no length is read back to the
host. Dense boolean masks, additive biases and score-modifying programs run on the eager fp32
path (`attention_reference`), which is also the CPU oracle; that is logged once.
"""

from __future__ import annotations

import math

import torch

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



# ---------------------------------------------------------------------------- segment bounds
def segment_bounds_from_cu_seqlens(cu_seqlens, total):
    """cu_seqlens [n + 1] (device) -> (seg_start, seg_end), int32 [total]: first token of each
    token's sequence and one past its last. Tokens beyond cu_seqlens[-1] form a tail segment."""
    cu = cu_seqlens.to(torch.int64)
    pos = torch.arange(total, device=cu.device)
    idx = torch.searchsorted(cu[1:].contiguous(), pos, right=True)
    n = cu.numel() - 1
    ext = torch.cat([cu, cu.new_full((1,), total)])
    start = ext[idx.clamp(max=n)]
    end = ext[(idx + 1).clamp(max=n + 1)]
    start = torch.where(idx >= n, cu[-1].expand_as(start), start)
    return start.to(torch.int32).contiguous(), end.to(torch.int32).contiguous()


def segment_bounds_from_offsets(document_offsets, seq_len):
    """document_offsets [B, n + 1] cumulative lengths per row (padded by repeating the end) ->
    flat (seg_start, seg_end) int32 [B * seq_len]; positions past a row's last offset form one
    trailing segment of that row."""
    off = document_offsets.to(torch.int64)
    B = off.shape[0]
    pos = torch.arange(seq_len, device=off.device)
    doc = (pos[None, :, None] >= off[:, None, 1:]).sum(-1)                    # [B, S]
    ext = torch.cat([off, off.new_full((B, 1), seq_len)], 1)
    start = torch.gather(ext, 1, doc)
    end = torch.gather(ext, 1, doc + 1)
    end = torch.where(end <= start, torch.full_like(end, seq_len), end)
    base = (torch.arange(B, device=off.device) * seq_len)[:, None]
    return (start + base).to(torch.int32).reshape(-1).contiguous(), \
        (end.clamp(max=seq_len) + base).to(torch.int32).reshape(-1).contiguous()


def segment_bounds_from_document_ids(document_ids):
    """document_ids [B, S] (equal ids are contiguous within a row) -> flat (seg_start, seg_end)."""
    B, S = document_ids.shape
    idx = torch.arange(B * S, device=document_ids.device).view(B, S)
    first = torch.ones(B, S, dtype=torch.bool, device=document_ids.device)
    first[:, 1:] = document_ids[:, 1:] != document_ids[:, :-1]
    last = torch.ones_like(first)
    last[:, :-1] = first[:, 1:]
    start = torch.cummax(torch.where(first, idx, idx.new_zeros(())), 1).values
    big = B * S + 1
    end = torch.cummin(torch.where(last, idx + 1, idx.new_full((), big)).flip(1), 1).values.flip(1)
    return start.to(torch.int32).reshape(-1).contiguous(), end.to(torch.int32).reshape(-1).contiguous()


_SEG_CACHE = {"key": None, "value": None}


def _cached_bounds(tensor, extra, build):
    """Segment bounds depend on a small index tensor that every layer of a step passes again:
    build them once per tensor version."""
    key = (id(tensor), tensor._version, tensor.data_ptr(), extra)
    if _SEG_CACHE["key"] != key:
        _SEG_CACHE["key"], _SEG_CACHE["value"] = key, build()
    return _SEG_CACHE["value"]


# ---------------------------------------------------------------------------- kernel front-end
def _heads_view(t):
    """[..., H, D] with adjacent heads and leading dims that collapse to one token stride."""
    D = t.shape[-1]
    ok = t.stride(-1) == 1 and t.stride(-2) == D and t.stride(-3) % 8 == 0 and t.data_ptr() % 16 == 0
    for d in range(t.dim() - 4, -1, -1):
        ok = ok and (t.shape[d] == 1 or t.stride(d) == t.stride(d + 1) * t.shape[d + 1])
    return t if ok else t.contiguous()


class _AttentionFn(torch.autograd.Function):
    """q [..., Hq, D], k / v [..., Hk, D] over the same tokens -> out shaped like q."""

    @staticmethod
    def forward(ctx, q, k, v, seg_start, seg_end, seq_len, causal, window, scale, softcap):
        C = ops.ext()
        q, k, v = _heads_view(q), _heads_view(k), _heads_view(v)
        out, lse = C.attention_fwd(q, k, v, seg_start, seg_end, seq_len, causal, window, scale, softcap,
                                   ops.status_word(q.device))
        ctx.save_for_backward(q, k, v, out, lse, seg_start, seg_end)
        ctx.cfg = (seq_len, causal, window, scale, softcap)
        return out

    @staticmethod
    def backward(ctx, dout):
        C = ops.ext()
        q, k, v, out, lse, seg_start, seg_end = ctx.saved_tensors
        seq_len, causal, window, scale, softcap = ctx.cfg
        dq = torch.empty(q.shape, device=q.device, dtype=q.dtype)
        dk = torch.empty(k.shape, device=k.device, dtype=k.dtype)
        dv = torch.empty(v.shape, device=v.device, dtype=v.dtype)
        C.attention_bwd(q, k, v, out, dout.contiguous(), lse, dq, dk, dv, seg_start, seg_end, seq_len, causal,
                        window, scale, softcap, ops.status_word(q.device))
        return dq, dk, dv, None, None, None, None, None, None, None


def _kernel_ok(q, k, v):
    return (ops.use_sm100(q) and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
            and q.shape[-1] in (64, 128) and k.shape[-1] == q.shape[-1] and v.shape[-1] == q.shape[-1]
            and q.shape[:-2] == k.shape[:-2] and q.shape[-2] % k.shape[-2] == 0)


_noted_eager = set()


def _note_eager(why):
    if why in _noted_eager:
        return
    _noted_eager.add(why)
    from halite_b200.logging import logger

    logger.warning(f"attention: {why}; running the eager fp32 path instead of the sm_100a kernel")


def attention(q, k, v, causal=True, scale=None, softcap=0.0, window=None, mask=None, bias=None,
              document_ids=None, cu_seqlens=None, max_seqlen=None, document_offsets=None, segments=None):
    """q [B, S, Hq, D]; k, v [B, S, Hk, D]. Packed input is [1, total, H, D] (or [total, H, D]) with
    `cu_seqlens`; per-row documents are given by `document_ids` [B, S] or `document_offsets`
    [B, n + 1]; `segments` = (seg_start, seg_end) passes ready-made bounds."""
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    softcap = float(softcap or 0.0)
    window_i = int(window) if window else 0
    if mask is None and bias is None and _kernel_ok(q, k, v):
        total = q.numel() // (q.shape[-1] * q.shape[-2])
        seq_len = q.shape[-3]
        if segments is None:
            if cu_seqlens is not None:
                segments = _cached_bounds(cu_seqlens, total, lambda: segment_bounds_from_cu_seqlens(cu_seqlens, total))
            elif document_offsets is not None:
                segments = _cached_bounds(document_offsets, seq_len,
                                          lambda: segment_bounds_from_offsets(document_offsets, seq_len))
            elif document_ids is not None:
                segments = _cached_bounds(document_ids, 0, lambda: segment_bounds_from_document_ids(document_ids))
        seg_start, seg_end = segments if segments is not None else (None, None)
        return _AttentionFn.apply(q, k, v, seg_start, seg_end, seq_len, bool(causal), window_i, scale, softcap)
    if q.is_cuda and not ops.force_reference():
        _note_eager("dense mask / additive bias" if (mask is not None or bias is not None)
                    else f"unsupported shape or dtype {tuple(q.shape)} x {tuple(k.shape)} {q.dtype}")
    if cu_seqlens is not None:
        return _varlen_reference(q, k, v, cu_seqlens, causal, scale, softcap, window)
    if document_offsets is not None and document_ids is None:
        S = q.shape[1]
        pos = torch.arange(S, device=q.device)
        document_ids = (pos[None, :, None] >= document_offsets[:, None, 1:]).sum(-1)
    return attention_reference(q, k, v, causal, scale, softcap, window, mask, bias, document_ids,
                               q_offset=None)


def _varlen_reference(q, k, v, cu_seqlens, causal, scale, softcap, window):
    """Eager oracle for packed sequences (reads the lengths on the host: CPU tests only)."""
    squeeze = q.dim() == 4
    if squeeze:
        q, k, v = q[0], k[0], v[0]
    bounds = cu_seqlens.tolist()
    outs = []
    for s, e in zip(bounds[:-1], bounds[1:]):
        outs.append(attention_reference(q[None, s:e], k[None, s:e], v[None, s:e], causal, scale, softcap, window,
                                        q_offset=None)[0])
    if bounds[-1] < q.shape[0]:
        outs.append(torch.zeros_like(q[bounds[-1]:]))
    out = torch.cat(outs, 0)
    return out[None] if squeeze else out


def varlen_attention(q, k, v, cu_seqlens, max_seqlen=None, causal=True, scale=None, softcap=0.0,
                     window=None):
    """Packed sequences: q,k,v [total, H, D] (or [1,total,H,D]); cu_seqlens [n+1] int."""
    return attention(q, k, v, causal, scale, softcap, window, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)


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
        out, lse = C.attention_fwd(q, k, v, None, None, S, causal, 0, scale, 0.0, ops.status_word(qkv.device))
        if ctx.needs_input_grad[0]:
            ctx.save_for_backward(qkv, out, lse)
            ctx.rope = (cos, sin, pos, interleaved)
            ctx.dims = (B, S, n_heads, n_kv, head_dim, causal, scale)
        return out.view(B, S, qd)

    @staticmethod
    def backward(ctx, dout):
        C = ops.ext()
        qkv, out, lse = ctx.saved_tensors
        B, S, H, Hk, D, causal, scale = ctx.dims
        qd, kd = H * D, Hk * D
        q = qkv[..., :qd].unflatten(-1, (H, D))
        k = qkv[..., qd:qd + kd].unflatten(-1, (Hk, D))
        v = qkv[..., qd + kd:].unflatten(-1, (Hk, D))
        dqkv = torch.empty_like(qkv)
        gq = dqkv[..., :qd].unflatten(-1, (H, D))
        gk = dqkv[..., qd:qd + kd].unflatten(-1, (Hk, D))
        gv = dqkv[..., qd + kd:].unflatten(-1, (Hk, D))
        cos, sin, pos, interleaved = ctx.rope
        rot = cos.shape[-1] * 2 if cos is not None else 0
        # dQ and dV land in their slots of the packed gradient straight from the kernels (dQ is
        # rotated back on its way out of the fp32 accumulator); dK goes there directly when nothing
        # has to be rotated, else through one inverse-rotation pass
        vec_ok = rot == 0 or rot % (8 if interleaved else 16) == 0
        dk = gk if rot == 0 else torch.empty(B, S, Hk, D, device=qkv.device, dtype=qkv.dtype)
        dq = gq if vec_ok else torch.empty(B, S, H, D, device=qkv.device, dtype=qkv.dtype)
        C.attention_bwd(q, k, v, out, dout.reshape(B, S, H, D).contiguous(), lse, dq, dk, gv, None, None, S,
                        causal, 0, scale, 0.0, ops.status_word(qkv.device),
                        cos if rot and vec_ok else None, sin if rot and vec_ok else None,
                        pos if rot and vec_ok else None, rot if vec_ok else 0, interleaved)
        if not vec_ok:
            C.rope_copy(dq, gq, cos, sin, pos, rot, interleaved, True)
        if rot:
            C.rope_copy(dk, gk, cos, sin, pos, rot, interleaved, True)
        return dqkv, None, None, None, None, None, None, None, None, None


def packed_qkv_attention(qkv, n_heads, n_kv_heads, head_dim, cos=None, sin=None, positions=None,
                         interleaved=True, causal=True, scale=None):
    """Attention over a packed QKV projection output (modified in place by RoPE)."""
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
    if ops.use_sm100(qkv) and qkv.is_contiguous() and head_dim in (64, 128) and qkv.shape[-1] % 8 == 0:
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
