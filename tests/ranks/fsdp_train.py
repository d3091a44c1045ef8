"""Rank script: 20 AdamW steps of the tiny Llama under the sharding layer (Gloo, CPU, fp32),
checked against a single-process plain-PyTorch replica that sees every rank's batch."""

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
mode = sys.argv[1] if len(sys.argv) > 1 else "fsdp"
# "<mode>_micro": every step's batch goes through in two micro-batches, the first one inside
# `no_sync()` (gradients only accumulate; one reduction per step); "<mode>_micro_sync" does the
# same without `no_sync()` (a reduction per micro-batch, which must still give the right sum)
micro = "_micro" in mode
hold_back = micro and not mode.endswith("_sync")
reshard = "_reshard" in mode      # memory-lean schedule: units are whole only around their own passes
mode = mode.split("_")[0]


def build():
    zoo = load_module(os.path.join(ROOT, "configs/models/transformer.py"))
    cfg = zoo.transformer(vocab_size=1024, dim=256, n_heads=4, head_dim=64, n_layers=4,
                          intermediate_size=688, context_len=512, n_key_value_heads=2,
                          rms_norm_epsilon=1e-5, qkv_split=True, gated_ff_split=True,
                          init=partial(torch.nn.init.normal_, std=0.02))
    torch.manual_seed(0)
    m = instantiate(cfg)
    m.init_weights()
    return m


ws = int(os.environ["WORLD_SIZE"])
if mode == "hsdp":
    pd = ParallelDims(dp_replicate=2, dp_shard=ws // 2)
elif mode == "ddp":
    pd = ParallelDims(dp_replicate=ws, dp_shard=1)
else:
    pd = ParallelDims(dp_shard=ws)
pd.build_mesh("cpu")
rank = pd.rank
steps = 20 if mode == "fsdp" and not micro else 6
g = torch.Generator().manual_seed(0)
data = torch.randint(0, 1024, (ws, steps, 4, 257), generator=g)
model, ref = build(), build()
model = parallelize(model, pd, pd, param_dtype="float32", reduce_dtype="float32", device="cpu",
                    reshard_after_forward=reshard)
if reshard:
    assert sum(u.reshard for u in model._hb_fsdp.units) == 4
opt = build_optimizer(partial(torch.optim.AdamW, lr=3e-4, betas=(0.9, 0.95)), model, weight_decay=0.1)
ropt = torch.optim.AdamW(group_parameters(ref, 0.1), lr=3e-4, betas=(0.9, 0.95))
worst = 0.0
for step in range(steps):
    x = data[rank, step]
    if micro:
        import contextlib

        loss = 0.0
        for i, xm in enumerate(x.chunk(2)):
            hold = model._hb_fsdp.no_sync() if hold_back and i == 0 else contextlib.nullcontext()
            with hold:
                lm = torch.nn.functional.cross_entropy(model(xm[:, :-1]).logits.flatten(0, 1),
                                                       xm[:, 1:].flatten()) / 2
                lm.backward()
            loss = loss + lm.detach()
    else:
        loss = torch.nn.functional.cross_entropy(model(x[:, :-1]).logits.flatten(0, 1), x[:, 1:].flatten())
        loss.backward()
    n = clip_grad_norm_(model, 1.0, opt)
    opt.step()
    opt.zero_grad()
    tot = 0.0
    for r in range(ws):
        xr = data[r, step]
        l = torch.nn.functional.cross_entropy(ref(xr[:, :-1]).logits.flatten(0, 1), xr[:, 1:].flatten()) / ws
        l.backward()
        tot += l.item()
    rn = torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
    ropt.step()
    ropt.zero_grad()
    lt = loss.detach().clone()
    dist.all_reduce(lt)
    worst = max(worst, abs(lt.item() / ws - tot), abs(n.item() - rn.item()))
if reshard:
    blocks = [u for u in model._hb_fsdp.units if u.reshard]
    # between steps a rank holds only its shard of every block, and no full gradient buffer
    assert all(u.full_param.untyped_storage().size() == 0 for u in blocks), "parameters were left gathered"
    assert all(u.full_grad.untyped_storage().size() == 0 for u in blocks), "gradient buffers were left allocated"
    model._hb_fsdp.wait_parameters()      # whole again for the comparison below
diff = max((a - b).abs().max().item() for a, b in zip(model.parameters(), ref.parameters()))
print(f"RESULT rank={rank} loss_norm_dev={worst:.3e} param_diff={diff:.3e} final_loss={tot:.4f}")
assert worst < 1e-4 and diff < 1e-4
dist.barrier()
dist.destroy_process_group()
