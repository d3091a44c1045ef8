"""Expert feed-forward over tokens sorted by expert (reference: transformers/moe/scattermoe/
scattermoe.py:9-102 and ops.py:279-462, whose Triton grouped GEMMs this replaces).

Tokens are sorted by expert once; each expert's contiguous row range then goes through the
sm_100a GEMM (`grouped_matmul`: forward `x_e @ W_e`, dgrad `dy_e @ W_e^T`, wgrad `x_e^T @ dy_e`,
all on operand layouts the kernel reads without transposes), the gate-weighted results are
scattered back with one index_add. On CPU the same function runs with `torch.matmul`.
"""

from __future__ import annotations

import torch
from torch import nn

import halite_b200.ops as ops
from halite_b200.models.initialize import init_weights
from halite_b200.ops.linear import gemm


def expert_boundaries(sorted_expert_indices, n_experts):
    """Cumulative end offset of every expert in the sorted order ([E] int64). Indices beyond
    `n_experts` (dropped slots sort last) are not counted."""
    valid = sorted_expert_indices < n_experts
    counts = torch.zeros(n_experts, dtype=torch.long, device=sorted_expert_indices.device)
    counts.scatter_add_(0, sorted_expert_indices[valid], torch.ones_like(sorted_expert_indices[valid]))
    return counts.cumsum(0)


def _use_kernel(x, w):
    return ops.use_sm100(x) and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and w.shape[-1] % 8 == 0


class _GroupedMatmul(torch.autograd.Function):
    """out[rows of expert e] = x[rows of expert e] @ weight[e]; weight [E, in, out]."""

    @staticmethod
    def forward(ctx, x, weight, bounds):
        ctx.save_for_backward(x, weight)
        ctx.bounds = bounds
        out = x.new_empty(x.shape[0], weight.shape[2])
        kernel = _use_kernel(x, weight)
        start = 0
        for e, end in enumerate(bounds):
            if end > start:
                if kernel:
                    gemm(x[start:end], weight[e], out=out[start:end], b_mn=True)
                else:
                    torch.matmul(x[start:end], weight[e], out=out[start:end])
            start = end
        if start < x.shape[0]:
            out[start:].zero_()          # dropped slots
        return out

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy = dy.contiguous()
        kernel = _use_kernel(x, weight)
        dx = torch.zeros_like(x) if ctx.needs_input_grad[0] else None
        dw = torch.zeros_like(weight) if ctx.needs_input_grad[1] else None
        start = 0
        for e, end in enumerate(ctx.bounds):
            if end > start:
                xs, ds = x[start:end], dy[start:end]
                if dx is not None:
                    if kernel:
                        gemm(ds, weight[e], out=dx[start:end])               # [m,out] @ [in,out]^T
                    else:
                        torch.matmul(ds, weight[e].t(), out=dx[start:end])
                if dw is not None:
                    if kernel:
                        gemm(xs, ds, out=dw[e], a_mn=True, b_mn=True)         # [m,in]^T @ [m,out]
                    else:
                        torch.matmul(xs.t(), ds, out=dw[e])
            start = end
        return dx, dw, None


def grouped_matmul(x, weight, bounds):
    """`bounds`: python list of cumulative end offsets per expert (from `expert_boundaries`)."""
    return _GroupedMatmul.apply(x, weight, list(bounds))


class ExpertLinear(nn.Module):
    def __init__(self, n_experts, in_features, out_features):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(n_experts, in_features, out_features))

    def forward(self, input, bounds):
        return grouped_matmul(input, self.weight, bounds)


class FeedForward(nn.Module):
    def __init__(self, linear1, activation, linear2, top_k, dropout=0, linear1_init=None, linear2_init=None):
        super().__init__()
        self.linear1, self.activation, self.linear2 = linear1, activation, linear2
        self.dropout = nn.Dropout(dropout)
        self.n_experts = linear1.weight.shape[0]
        self.top_k = top_k
        self.linear1_init, self.linear2_init = linear1_init, linear2_init

    def init_weights(self):
        for lin, fn in ((self.linear1, self.linear1_init), (self.linear2, self.linear2_init)):
            if fn is not None:
                for e in range(self.n_experts):
                    fn(lin.weight.data[e].t())      # initialisers see [out, in], as for nn.Linear
            else:
                nn.init.normal_(lin.weight, std=0.02)

    def forward(self, input, expert_probs, expert_indices):
        shape = input.shape
        x = input.reshape(-1, shape[-1])
        with torch.no_grad():
            flat = expert_indices.reshape(-1)
            sorted_experts, order = flat.sort(stable=True)
            bounds = expert_boundaries(sorted_experts, self.n_experts).tolist()   # the one host sync
            n_kept = bounds[-1]
            order = order[:n_kept]
            token = order // expert_indices.shape[1]
        gathered = x.index_select(0, token)                       # expert-contiguous rows
        hidden = self.dropout(self.activation(self.linear1(gathered, bounds)))
        out = self.linear2(hidden, bounds)
        gates = expert_probs.reshape(-1)[order].unsqueeze(-1).to(out.dtype)
        combined = torch.zeros(x.shape[0], out.shape[-1], dtype=out.dtype, device=out.device)
        combined = combined.index_add(0, token, out * gates)
        return combined.view(*shape[:-1], out.shape[-1])
