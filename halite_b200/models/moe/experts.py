"""Expert feed-forward over tokens sorted by expert (reference: transformers/moe/scattermoe/
scattermoe.py:9-102 and ops.py:279-462, whose Triton grouped GEMMs this replaces).

Tokens are sorted by expert once; each expert's contiguous row range then goes through the
sm_100a GEMM (`grouped_matmul`: forward `x_e @ W_e`, dgrad `dy_e @ W_e^T`, wgrad `x_e^T @ dy_e`,
all on operand layouts the kernel reads without transposes), the gate-weighted results are
scattered back with one index_add. On CPU the same function runs with `torch.matmul`.

On sm_100a the whole layer runs without a host round trip: every expert's rows are placed in a
block padded to a multiple of 128 rows (`PaddedLayout`, computed with device ops only, sized for
the worst case), so each 128-row tile belongs to one expert and the grouped modes of the GEMM
kernel take their tile table (`tile_group`) and per-expert K ranges from device memory: one
launch per projection for forward and dgrad, one for all experts' wgrads.
"""

from __future__ import annotations

import torch
from torch import nn

import halite_b200.ops as ops
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


_TILE = 128


class PaddedLayout:
    """Where each (token, slot) pair sits in the expert-major, 128-row padded buffer. Everything
    is a device tensor; sizes depend only on the static shapes."""

    def __init__(self, expert_indices, n_experts):
        flat = expert_indices.reshape(-1)
        n_slots = flat.numel()
        dev = flat.device
        self.rows = n_slots + _TILE * n_experts                 # worst case: every expert padded by < 128
        self.rows = (self.rows + _TILE - 1) // _TILE * _TILE
        sorted_experts, order = flat.sort(stable=True)
        valid = sorted_experts < n_experts                      # dropped slots carry an id >= n_experts
        e = sorted_experts.clamp(max=n_experts - 1)
        counts = torch.zeros(n_experts, dtype=torch.long, device=dev).scatter_add_(0, e, valid.long())
        padded = (counts + _TILE - 1) // _TILE * _TILE
        p_end = padded.cumsum(0)
        p_start = p_end - padded
        start = counts.cumsum(0) - counts
        slot = torch.arange(n_slots, device=dev)
        dest = p_start[e] + (slot - start[e])
        self.dest = torch.where(valid, dest, torch.full_like(dest, self.rows))     # dropped slots -> spare row
        self.valid = valid
        self.token = order // expert_indices.shape[1]
        self.order = order
        tiles = torch.arange(self.rows // _TILE, device=dev)
        group = torch.searchsorted(p_end // _TILE, tiles, right=True)
        # position of every (token, slot) pair in token-major order: a permutation of the valid rows,
        # so moving rows in and out of the padded buffer needs copies, never atomic adds
        self.pos = torch.empty_like(self.dest).index_copy_(0, order, self.dest)
        self.valid_slot = torch.empty_like(valid).index_copy_(0, order, valid)
        self.top_k = expert_indices.shape[1]
        self.tile_group = torch.where(group < n_experts, group, torch.full_like(group, -1)).int().contiguous()
        self.k_begin = p_start.int().contiguous()
        self.k_end = p_end.int().contiguous()
        self.n_experts = n_experts


class _ScatterRows(torch.autograd.Function):
    """padded[pos[t * k + j]] = x[t] for every slot j of token t (dropped slots land in the spare
    last row); backward gathers the k rows of each token and adds them."""

    @staticmethod
    def forward(ctx, x, layout):
        T, D = x.shape
        k = layout.top_k
        padded = torch.zeros(layout.rows + 1, D, dtype=x.dtype, device=x.device)
        padded.index_copy_(0, layout.pos, x.unsqueeze(1).expand(T, k, D).reshape(T * k, D))
        padded[layout.rows].zero_()
        ctx.layout = layout
        return padded

    @staticmethod
    def backward(ctx, g):
        lay = ctx.layout
        picked = g.index_select(0, lay.pos) * lay.valid_slot.unsqueeze(-1).to(g.dtype)
        return picked.view(-1, lay.top_k, g.shape[-1]).sum(1), None


class _GatherRows(torch.autograd.Function):
    """rows[t * k + j] = out[pos[t * k + j]] (zeros for dropped slots); backward copies each
    gradient row back to its unique position."""

    @staticmethod
    def forward(ctx, out, layout):
        ctx.layout = layout
        ctx.n_rows = out.shape[0]
        picked = out.index_select(0, layout.pos.clamp(max=out.shape[0] - 1))
        return picked * layout.valid_slot.unsqueeze(-1).to(out.dtype)

    @staticmethod
    def backward(ctx, g):
        lay = ctx.layout
        grad = torch.zeros(ctx.n_rows + 1, g.shape[-1], dtype=g.dtype, device=g.device)
        grad.index_copy_(0, lay.pos, g * lay.valid_slot.unsqueeze(-1).to(g.dtype))
        return grad[: ctx.n_rows], None


class _GroupedMatmulPadded(torch.autograd.Function):
    """out[rows of expert e] = x[rows of expert e] @ weight[e] on the padded layout, one launch;
    backward: one launch for dx, one for every expert's dw."""

    @staticmethod
    def forward(ctx, x, weight, layout):
        E, k_in, k_out = weight.shape
        out = torch.zeros(x.shape[0], k_out, device=x.device, dtype=x.dtype)   # skipped tiles stay zero
        gemm(x, weight.view(E * k_in, k_out), out=out, b_mn=True,
             group=dict(mode=1, tile_group_ptr=layout.tile_group.data_ptr(), b_group_rows=k_in,
                        b_total_rows=E * k_in))
        ctx.save_for_backward(x, weight)
        ctx.layout = layout
        return out

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        layout = ctx.layout
        E, k_in, k_out = weight.shape
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.zeros_like(x)
            gemm(dy, weight.view(E * k_in, k_out), out=dx,
                 group=dict(mode=1, tile_group_ptr=layout.tile_group.data_ptr(), b_group_rows=k_in,
                            b_total_rows=E * k_in))
        if ctx.needs_input_grad[1]:
            dw = torch.zeros_like(weight)                       # experts without tokens keep zeros
            gemm(x, dy, out=dw, a_mn=True, b_mn=True,
                 group=dict(mode=2, n_groups=E, k_begin_ptr=layout.k_begin.data_ptr(),
                            k_end_ptr=layout.k_end.data_ptr(), d_group_elems=k_in * k_out))
        return dx, dw, None


def _padded_ok(x, w1, w2):
    return (_use_kernel(x, w1) and w1.shape[1] % 64 == 0 and w1.shape[2] % 64 == 0 and w2.shape[1] % 64 == 0 and w2.shape[2] % 64 == 0
            and w1.is_contiguous() and w2.is_contiguous() and not ops.force_reference())


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
        if _padded_ok(x, self.linear1.weight, self.linear2.weight):
            return self._forward_padded(x, expert_probs, expert_indices).view(*shape[:-1], -1)
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

    def _forward_padded(self, x, expert_probs, expert_indices):
        """The layer without a host round trip (see `PaddedLayout`). Padding rows, rows past the
        last expert and the spare row hold zeros throughout."""
        with torch.no_grad():
            lay = PaddedLayout(expert_indices, self.n_experts)
        body = _ScatterRows.apply(x, lay)[: lay.rows]
        hidden = self.dropout(self.activation(_GroupedMatmulPadded.apply(body, self.linear1.weight, lay)))
        out = _GroupedMatmulPadded.apply(hidden, self.linear2.weight, lay)
        rows = _GatherRows.apply(out, lay)                         # token-major: [tokens * k, dim]
        gates = expert_probs.reshape(-1, 1).to(out.dtype)
        return (rows * gates).view(x.shape[0], lay.top_k, -1).sum(1)
