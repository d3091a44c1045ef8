"""Gated activations `act(gate) * up` (SwiGLU, GEGLU-tanh), forward and backward in one pass
each. `gated_act_packed` takes the output of one fused gate/up projection ([..., 2*I]) and
returns the gradient as one [..., 2*I] tensor, so the dgrad / wgrad GEMMs that follow see a
single operand and autograd never zero-fills slices."""

from __future__ import annotations

import torch
import torch.nn.functional as F

import halite_b200.ops as ops

_KINDS = {"silu": 0, "gelu_tanh": 1}


def _ref(gate, up, kind):
    if kind == "silu":
        return F.silu(gate) * up
    return F.gelu(gate, approximate="tanh") * up


class _GatedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up, kind):
        ctx.save_for_backward(gate, up)
        ctx.kind = kind
        return ops.ext().gated_act_fwd(gate, up, kind)

    @staticmethod
    def backward(ctx, dout):
        gate, up = ctx.saved_tensors
        dg, du = ops.ext().gated_act_bwd(gate, up, dout.contiguous(), ctx.kind, None, None)
        return dg.view(gate.shape), du.view(up.shape), None


class _GatedPackedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, packed, kind, gate_first):
        half = packed.shape[-1] // 2
        p2 = packed.reshape(-1, 2 * half)
        gate, up = (p2[:, :half], p2[:, half:]) if gate_first else (p2[:, half:], p2[:, :half])
        ctx.save_for_backward(p2)
        ctx.kind, ctx.gate_first, ctx.shape = kind, gate_first, packed.shape
        out = ops.ext().gated_act_fwd(gate, up, kind)
        return out.view(*packed.shape[:-1], half)

    @staticmethod
    def backward(ctx, dout):
        (p2,) = ctx.saved_tensors
        half = p2.shape[-1] // 2
        gate, up = (p2[:, :half], p2[:, half:]) if ctx.gate_first else (p2[:, half:], p2[:, :half])
        dp = torch.empty_like(p2)
        dg, du = (dp[:, :half], dp[:, half:]) if ctx.gate_first else (dp[:, half:], dp[:, :half])
        ops.ext().gated_act_bwd(gate, up, dout.reshape(-1, half).contiguous(), ctx.kind, dg, du)
        return dp.view(ctx.shape), None, None


def gated_act(gate, up, kind="silu"):
    if ops.use_sm100(gate) and gate.shape[-1] % 8 == 0 and gate.stride(-1) == 1 and up.stride(-1) == 1:
        return _GatedFn.apply(gate, up, _KINDS[kind])
    return _ref(gate, up, kind)


def gated_act_packed(packed, kind="silu", gate_first=True):
    """packed[..., 2*I] = concat(gate, up) (or (up, gate) when not gate_first) -> [..., I]."""
    half = packed.shape[-1] // 2
    if ops.use_sm100(packed) and half % 8 == 0 and packed.is_contiguous():
        return _GatedPackedFn.apply(packed, _KINDS[kind], gate_first)
    a, b = packed[..., :half], packed[..., half:]
    gate, up = (a, b) if gate_first else (b, a)
    return _ref(gate, up, kind)


def swiglu(gate, up):
    return gated_act(gate, up, "silu")


def geglu_tanh(gate, up):
    return gated_act(gate, up, "gelu_tanh")
