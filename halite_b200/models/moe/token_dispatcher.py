"""Expert-parallel token exchange (reference: transformers/moe/token_dispatcher.py:56-330).

Experts are split evenly over the ranks of `ep_group`. Per layer: tokens are sorted by global
expert, the per-(rank, local expert) counts are exchanged, one all-to-all moves the rows to the
ranks that own their experts, rows are regrouped by local expert, the local experts run, and
the same path runs backwards. The all-to-all is differentiable.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from halite_b200.models.moe.experts import grouped_matmul


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty(sum(out_splits), *x.shape[1:])
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        back = grad.new_empty(sum(ctx.in_splits), *grad.shape[1:])
        dist.all_to_all_single(back, grad.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return back, None, None, None


class AlltoAllTokenDispatcher(nn.Module):
    def __init__(self, n_experts, capacity_factor=None, pad_to_capacity=False, deterministic=False):
        super().__init__()
        self.n_experts = n_experts
        self.capacity_factor, self.pad_to_capacity, self.deterministic = capacity_factor, pad_to_capacity, deterministic
        self.active = False

    def parallelize(self, ep_group):
        self.ep_group = ep_group
        self.ep_size = dist.get_world_size(ep_group)
        self.ep_rank = dist.get_rank(ep_group)
        if self.n_experts % self.ep_size:
            raise ValueError("n_experts must be divisible by the expert-parallel size")
        self.n_local_experts = self.n_experts // self.ep_size
        self.active = self.ep_size > 1

    def forward(self, inputs, probs, indices, experts):
        shape = inputs.shape
        x = inputs.reshape(-1, shape[-1])
        E, L, W = self.n_experts, self.n_local_experts, self.ep_size
        with torch.no_grad():
            flat = indices.reshape(-1)
            sorted_experts, order = flat.sort(stable=True)
            counts = torch.zeros(E, dtype=torch.long, device=x.device)
            valid = sorted_experts < E
            counts.scatter_add_(0, sorted_experts[valid], torch.ones_like(sorted_experts[valid]))
            order = order[: int(counts.sum())]
            token = order // indices.shape[1]
            # counts[r*L + l] rows go to rank r, local expert l; learn what every rank sends me
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts, group=self.ep_group)      # [W, L] by source rank
            in_splits = counts.view(W, L).sum(1).tolist()
            recv = recv_counts.view(W, L)
            out_splits = recv.sum(1).tolist()
            # received rows arrive source-major; regroup them expert-major
            seg = recv.reshape(-1)
            src_of = torch.repeat_interleave(torch.arange(W * L, device=x.device), seg)
            regroup = torch.sort((src_of % L) * W + src_of // L, stable=True)[1]
            bounds = recv.sum(0).cumsum(0).tolist()
        send = x.index_select(0, token)
        got = _AllToAll.apply(send, out_splits, in_splits, self.ep_group)
        local = got.index_select(0, regroup)
        w1 = experts.linear1.weight[self.ep_rank * L:(self.ep_rank + 1) * L] if experts.linear1.weight.shape[0] == E \
            else experts.linear1.weight
        w2 = experts.linear2.weight[self.ep_rank * L:(self.ep_rank + 1) * L] if experts.linear2.weight.shape[0] == E \
            else experts.linear2.weight
        hidden = experts.dropout(experts.activation(grouped_matmul(local, w1, bounds)))
        out_local = grouped_matmul(hidden, w2, bounds)
        undo = torch.empty_like(regroup)
        undo[regroup] = torch.arange(regroup.numel(), device=regroup.device)
        back = _AllToAll.apply(out_local.index_select(0, undo), in_splits, out_splits, self.ep_group)
        gates = probs.reshape(-1)[order].unsqueeze(-1).to(back.dtype)
        combined = torch.zeros(x.shape[0], back.shape[-1], dtype=back.dtype, device=back.device)
        combined = combined.index_add(0, token, back * gates)
        return combined.view(*shape[:-1], back.shape[-1])
