"""Rotary position embedding: table construction (incl. Llama-3 frequency scaling) and the
in-place sm_100a kernel with its conjugate backward.

Replaces the Triton rotary kernel of the reference (transformers/ops/rotary.py:14) and the
complex-multiply eager path (transformers/position.py:294-300).
"""

from __future__ import annotations

import math

import torch

import halite_b200.ops as ops


def rope_tables(inv_freq: torch.Tensor, max_pos: int, device=None):
    """cos/sin tables [max_pos, dim/2] in fp32, computed once on the host side in fp32."""
    t = torch.arange(max_pos, dtype=torch.float32, device=inv_freq.device)
    freqs = torch.outer(t, inv_freq.float())
    cos, sin = freqs.cos(), freqs.sin()
    if device is not None:
        cos, sin = cos.to(device), sin.to(device)
    return cos.contiguous(), sin.contiguous()


def llama3_scale_inv_freq(inv_freq, scale_factor=8, low_freq_factor=1, high_freq_factor=4,
                          original_context_len=8192):
    """Llama-3 long-context scaling: long wavelengths are slowed by `scale_factor`, short ones
    kept, the band in between is blended linearly in 1/wavelength."""
    low_wavelen = original_context_len / low_freq_factor
    high_wavelen = original_context_len / high_freq_factor
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_wavelen, inv_freq / scale_factor, inv_freq)
    smooth = (original_context_len / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
    blended = (1 - smooth) * scaled / scale_factor + smooth * scaled
    medium = (wavelen >= high_wavelen) & (wavelen <= low_wavelen)
    return torch.where(medium, blended, scaled)


def apply_rope_reference(x, cos, sin, positions, interleaved: bool):
    """x: [..., tokens..., heads, head_dim]; positions broadcastable to the token dims."""
    c = cos[positions].unsqueeze(-2)
    s = sin[positions].unsqueeze(-2)
    rot = cos.shape[-1] * 2
    xf = x.float()
    xr, rest = xf[..., :rot], xf[..., rot:]
    if interleaved:
        a, b = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack((a * c - b * s, a * s + b * c), -1).flatten(-2)
    else:
        a, b = xr[..., : rot // 2], xr[..., rot // 2:]
        out = torch.cat((a * c - b * s, b * c + a * s), -1)
    if rest.shape[-1]:
        out = torch.cat((out, rest), -1)
    return out.type_as(x)


class _RopeFn(torch.autograd.Function):
    """Rotates q and k in place (the projections' outputs are not needed un-rotated)."""

    @staticmethod
    def forward(ctx, q, k, cos, sin, positions, interleaved):
        C = ops.ext()
        rot = cos.shape[-1] * 2
        pos = positions.contiguous()
        C.rope_(q, cos, sin, pos, rot, interleaved, False)
        C.rope_(k, cos, sin, pos, rot, interleaved, False)
        ctx.save_for_backward(cos, sin, pos)
        ctx.interleaved = interleaved
        ctx.mark_dirty(q, k)
        return q, k

    @staticmethod
    def backward(ctx, dq, dk):
        cos, sin, pos = ctx.saved_tensors
        C = ops.ext()
        rot = cos.shape[-1] * 2
        # incoming gradients must not be modified in place: rotate packed copies
        dq = dq.clone(memory_format=torch.contiguous_format)
        dk = dk.clone(memory_format=torch.contiguous_format)
        C.rope_(dq, cos, sin, pos, rot, ctx.interleaved, True)
        C.rope_(dk, cos, sin, pos, rot, ctx.interleaved, True)
        return dq, dk, None, None, None, None


def _packed(t):
    return t.stride(-1) == 1 and t.stride(-2) == t.shape[-1]


def apply_rope(q, k, cos, sin, positions, interleaved: bool):
    """Rotate q [.., Hq, D] and k [.., Hk, D] by the table rows at `positions` (one per token).

    The sm_100a path works in place on views (e.g. slices of a fused QKV projection output).
    """
    if ops.use_sm100(q) and cos.dtype == torch.float32 and cos.is_cuda:
        ntok = q.numel() // (q.shape[-1] * q.shape[-2])
        pos = positions
        if pos.numel() != ntok:
            pos = pos.expand(q.shape[:-2]).contiguous()
        if not _packed(q):
            q = q.contiguous()
        if not _packed(k):
            k = k.contiguous()
        return _RopeFn.apply(q, k, cos, sin, pos.reshape(-1), interleaved)
    return (apply_rope_reference(q, cos, sin, positions, interleaved),
            apply_rope_reference(k, cos, sin, positions, interleaved))
