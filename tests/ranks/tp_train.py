"""Rank script: tensor-parallel (+ sharded data-parallel) training of the tiny Llama on CPU / Gloo
against a single-process replica. argv: tp size."""

import os
import sys
from functools import partial

import torch
import torch.distributed as dist

from halite_b200.conf import instantiate
from halite_b200.conf.loader import load_module
from halite_b200.optim import build_optimizer, group_parameters
from halite_b200.optim.sharded_adamw import clip_grad_norm_
from halite_b200.parallel import ParallelDims, parallelize

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
tp_size = int(sys.argv[1])
qkv_split = sys.argv[2] == "split" if len(sys.argv) > 2 else True


def build(fused_head):
    zoo = load_module(os.path.join(ROOT, "configs/models/transformer.py"))
    cfg = zoo.transformer(vocab_size=1024, dim=256, n_heads=4, head_dim=64, n_layers=2,
                          intermediate_size=512, context_len=512, n_key_value_heads=2,
                          rms_norm_epsilon=1e-5, qkv_split=qkv_split, gated_ff_split=qkv_split,
                          init=partial(torch.nn.init.normal_, std=0.02))
    if fused_head:
        cfg = zoo.use_fused_linear_cross_entropy(cfg)
    torch.manual_seed(0)
    m = instantiate(cfg)
    m.init_weights()
    return m


ws = int(os.environ["WORLD_SIZE"])
pd = ParallelDims(dp_shard=ws // tp_size, tp=tp_size)
pd.build_mesh("cpu")
rank, dp_rank, dp = pd.rank, pd.dp_rank, pd.dp
steps = 5
g = torch.Generator().manual_seed(0)
data = torch.randint(0, 1024, (dp, steps, 2, 65), generator=g)
model, ref = build(True), build(False)
model = parallelize(model, pd, pd, param_dtype="float32", reduce_dtype="float32", device="cpu")
opt = build_optimizer(partial(torch.optim.AdamW, lr=1e-3, betas=(0.9, 0.95)), model, weight_decay=0.1)
ropt = torch.optim.AdamW(group_parameters(ref, 0.1), lr=1e-3, betas=(0.9, 0.95))
worst = 0.0
for step in range(steps):
    x = data[dp_rank, step]
    out = model(x[:, :-1], target=x[:, 1:])
    out.loss.backward()
    n = clip_grad_norm_(model, 1.0, opt)
    opt.step()
    opt.zero_grad()
    tot = 0.0
    for r in range(dp):
        xr = data[r, step]
        l = torch.nn.functional.cross_entropy(ref(xr[:, :-1]).logits.flatten(0, 1), xr[:, 1:].flatten()) / dp
        l.backward()
        tot += l.item()
    rn = torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
    ropt.step()
    ropt.zero_grad()
    lt = out.loss.detach().clone()
    dist.all_reduce(lt)
    worst = max(worst, abs(lt.item() / ws - tot))
    # the norm reported by the sharded path covers this TP rank's parameter shard only
logits = model(data[0, 0][:, :-1]).logits
ref_logits = ref(data[0, 0][:, :-1]).logits
dev = (logits - ref_logits).abs().max().item()
print(f"RESULT rank={rank} loss_dev={worst:.3e} logits_dev={dev:.3e}")
assert worst < 2e-4 and dev < 2e-3, (worst, dev)
dist.barrier()
dist.destroy_process_group()
