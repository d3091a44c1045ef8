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
    """Out-of-place rotation of one [.., H, D] tensor (possibly a strided slice of a fused
    projection output) into a packed result; the backward pass rotates the gradient back."""

    @staticmethod
    def forward(ctx, x, cos, sin, pos, interleaved):
        C = ops.ext()
        out = torch.empty(x.shape, device=x.device, dtype=x.dtype)
        C.rope_copy(_collapsible(x), out, cos, sin, pos, cos.shape[-1] * 2, interleaved, False)
        ctx.save_for_backward(cos, sin, pos)
        ctx.interleaved = interleaved
        return out

    @staticmethod
    def backward(ctx, dx):
        cos, sin, pos = ctx.saved_tensors
        C = ops.ext()
        out = torch.empty(dx.shape, device=dx.device, dtype=dx.dtype)
        C.rope_copy(_collapsible(dx), out, cos, sin, pos, cos.shape[-1] * 2, ctx.interleaved, True)
        return out, None, None, None, None


def _collapsible(t):
    """`t` itself when its heads are packed and its leading dims fold into one token stride."""
    if not _packed(t):
        return t.contiguous()
    for d in range(t.dim() - 4, -1, -1):
        if t.shape[d] != 1 and t.stride(d) != t.stride(d + 1) * t.shape[d + 1]:
            return t.contiguous()
    return t


def _packed(t):
    return t.stride(-1) == 1 and t.stride(-2) == t.shape[-1]


def apply_rope(q, k, cos, sin, positions, interleaved: bool):
    """Rotate q [.., Hq, D] and k [.., Hk, D] by the table rows at `positions` (one per token).

    On sm_100a: out of place when a gradient is needed, else in place on the views (e.g. slices of
    a fused QKV projection output).
    """
    if ops.use_sm100(q) and cos.dtype == torch.float32 and cos.is_cuda:
        ntok = q.numel() // (q.shape[-1] * q.shape[-2])
        pos = positions
        if pos.numel() != ntok:
            pos = pos.expand(q.shape[:-2]).contiguous()
        pos = pos.reshape(-1).contiguous()
        if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad):
            return (_RopeFn.apply(q, cos, sin, pos, interleaved), _RopeFn.apply(k, cos, sin, pos, interleaved))
        # nothing to differentiate: rotate in place (on packed copies when the views are not packed)
        q, k = _collapsible(q), _collapsible(k)
        C = ops.ext()
        rot = cos.shape[-1] * 2
        C.rope_(q, cos, sin, pos, rot, interleaved, False)
        C.rope_(k, cos, sin, pos, rot, interleaved, False)
        return q, k
    return (apply_rope_reference(q, cos, sin, positions, interleaved),
            apply_rope_reference(k, cos, sin, positions, interleaved))
