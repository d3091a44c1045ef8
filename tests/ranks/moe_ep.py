"""Rank script: expert parallelism over Gloo. Every rank holds all expert weights (same seed);
the dispatcher routes each token to the rank that owns its expert. Output and input gradient
must equal the single-process layer; weight gradients must be non-zero only on owned experts
and, summed over ranks, equal the single-process gradients."""

import os

import torch
import torch.distributed as dist

from halite_b200.models.moe import AlltoAllTokenDispatcher, ExpertLinear, FeedForward, MoE, TopKRouter
from halite_b200.nn.activation import SwiGLU

dist.init_process_group("gloo")
rank, ws = dist.get_rank(), dist.get_world_size()
E, k, d, h = 4, 2, 16, 24


def make(dispatcher):
    torch.manual_seed(0)
    m = MoE(TopKRouter(d, E, k, pre_softmax=True, deterministic=True), dispatcher,
            FeedForward(ExpertLinear(E, d, 2 * h), SwiGLU(), ExpertLinear(E, h, d), top_k=k))
    for mod in m.modules():
        if hasattr(mod, "init_weights"):
            mod.init_weights()
    return m


ref, ep = make(None), make(AlltoAllTokenDispatcher(E))
ep.parallelize(dist.group.WORLD)
torch.manual_seed(100 + rank)
x = torch.randn(2, 7, d)
xr, xe = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
yr, _ = ref(xr)
ye, _ = ep(xe)
out_diff = (yr - ye).abs().max().item()
yr.square().sum().backward()
ye.square().sum().backward()
in_diff = (xr.grad - xe.grad).abs().max().item()
# weight grads: the reference on rank r only saw rank r's tokens; sum both sides over ranks
L = E // ws
g_ref = ref.experts.linear1.weight.grad.clone()
g_ep = ep.experts.linear1.weight.grad.clone()
owned = g_ep[rank * L:(rank + 1) * L].abs().sum().item()
other = g_ep.abs().sum().item() - owned
dist.all_reduce(g_ref)
dist.all_reduce(g_ep)
w_diff = (g_ref - g_ep).abs().max().item()
print(f"RESULT rank={rank} out={out_diff:.2e} dx={in_diff:.2e} dw={w_diff:.2e} owned={owned:.3f} other={other:.3f}")
assert out_diff < 1e-5 and in_diff < 1e-5 and w_diff < 1e-4 and owned > 0 and other == 0
dist.barrier()
dist.destroy_process_group()
