"""Rank script: train, checkpoint, keep training; then restore into a fresh model (optionally on
a different world size) and check that the continued run reproduces the same parameters."""

import os
import sys
from functools import partial

import torch
import torch.distributed as dist

from halite_b200.conf import instantiate
from halite_b200.conf.loader import load_module
from halite_b200.distributed.checkpoint import CheckpointManager
from halite_b200.optim import build_optimizer
from halite_b200.optim.lr_scheduler import cycle_scheduler
from halite_b200.optim.sharded_adamw import clip_grad_norm_
from halite_b200.parallel import ParallelDims, parallelize

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
directory, phase = sys.argv[1], sys.argv[2]


def build(seed):
    zoo = load_module(os.path.join(ROOT, "configs/models/transformer.py"))
    cfg = zoo.transformer(vocab_size=512, dim=128, n_heads=4, head_dim=32, n_layers=2,
                          intermediate_size=344, context_len=256, n_key_value_heads=2,
                          rms_norm_epsilon=1e-5, qkv_split=True, gated_ff_split=True,
                          init=partial(torch.nn.init.normal_, std=0.02))
    torch.manual_seed(seed)
    m = instantiate(cfg)
    m.init_weights()
    return m


ws = int(os.environ["WORLD_SIZE"])
pd = ParallelDims(dp_shard=ws)
pd.build_mesh("cpu")
g = torch.Generator().manual_seed(0)
data = torch.randint(0, 512, (8, 4, 65), generator=g)     # [step, global batch, tokens]


def make(seed):
    model = parallelize(build(seed), pd, pd, param_dtype="float32", reduce_dtype="float32", device="cpu")
    opt = build_optimizer(partial(torch.optim.AdamW, lr=1e-3, betas=(0.9, 0.95)), model, weight_decay=0.1)
    sched = cycle_scheduler(opt, lr=1e-3, n_iter=8, warmup=2, decay=("linear", "cos"))
    mgr = CheckpointManager(model, opt, sched, directory=directory, interval=2, keep_latest_k=2,
                            async_mode="async" if phase == "save_async" else "disabled")
    return model, opt, sched, mgr


def train(model, opt, sched, mgr, start, stop):
    per = data.shape[1] // ws
    for step in range(start, stop):
        x = data[step, pd.rank * per:(pd.rank + 1) * per]
        loss = torch.nn.functional.cross_entropy(model(x[:, :-1]).logits.flatten(0, 1), x[:, 1:].flatten())
        loss.backward()
        clip_grad_norm_(model, 1.0, opt)
        opt.step()
        sched.step()
        opt.zero_grad()
        if mgr is not None:
            mgr.save(step + 1)


def flat(model):
    return torch.cat([p.detach().flatten() for p in model.parameters()])


if phase.startswith("save"):
    model, opt, sched, mgr = make(0)
    train(model, opt, sched, mgr, 0, 6)       # saves at 2, 4, 6; keep_latest_k prunes step-2
    mgr._wait()
    dist.barrier()
    if pd.rank == 0:
        kept = sorted(os.listdir(directory))
        assert kept == ["step-4", "step-6"], kept
        torch.save(flat(model), os.path.join(directory, "final.pt"))
        # restore step 4 into a differently initialised model and replay steps 4, 5
    model2, opt2, sched2, mgr2 = make(123)
    assert mgr2.load(4)
    assert opt2._step == 4 and sched2.n_step == 4, (opt2._step, sched2.n_step)
    train(model2, opt2, sched2, None, 4, 6)
    diff = (flat(model2) - flat(model)).abs().max().item()
    print(f"RESULT rank={pd.rank} replay_diff={diff:.3e}")
    assert diff < 1e-6
else:
    # a different world size resumes from the newest step and must land on the same weights
    model, opt, sched, mgr = make(7)
    assert mgr.load(-1)
    want = torch.load(os.path.join(directory, "final.pt"))
    diff = (flat(model) - want).abs().max().item()
    print(f"RESULT rank={pd.rank} reshard_diff={diff:.3e} step={opt._step}")
    assert diff < 1e-6 and opt._step == 6
    train(model, opt, sched, None, 6, 8)
dist.barrier()
dist.destroy_process_group()
