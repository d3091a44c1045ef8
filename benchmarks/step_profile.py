"""Per-kernel time breakdown of one training step of the benchmark model:

    python -m benchmarks.step_profile [--layers 8] [--batch 8] [--seq 4096] [--rows 30]

Runs a few warm-up steps, then one step under `torch.profiler` (CUPTI kernel timestamps) and
prints device time per kernel name, largest first, with each kernel's share. Use it to decide
what to optimise; absolute step times come from `bench.py`, never from a profiled run.
"""

from __future__ import annotations

import argparse
import os
from functools import partial

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--conf", default=None, help="model config (default: the Llama-3.2-3B bench config)")
    ap.add_argument("--layers", type=int, default=8, help="keep only the first N blocks (0 = all)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--rows", type=int, default=30)
    args = ap.parse_args(argv)

    from torch.profiler import ProfilerActivity, profile

    from halite_b200.conf import instantiate, load_config
    from halite_b200.optim import build_optimizer
    from halite_b200.parallel import ParallelDims, parallelize
    from halite_b200.projects.common.train_fn import optimization_step

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    conf = load_config(args.conf or os.path.join(root, "configs/models/llama/llama3_2_3b_bench.py"))
    if args.layers:
        conf.model.blocks = conf.model.blocks[: args.layers]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    pd = ParallelDims(dp_shard=1, world_size=1)
    pd.build_mesh("cuda")
    with torch.device("meta"):
        model = instantiate(conf.model)
    model = parallelize(model, pd, pd, device=dev)
    model.init_weights(dev)
    opt = build_optimizer(partial(torch.optim.AdamW, lr=3e-4, betas=(0.9, 0.95)), model, weight_decay=0.1)
    vocab = model.embedding.embed_weight.shape[0]
    tok = torch.randint(0, vocab, (args.batch, args.seq + 1), device=dev)

    def step():
        return optimization_step(model, {"input": tok[:, :-1], "target": tok[:, 1:]}, opt, clip_grad_norm=1.0,
                                 calc_loss_in_model=True)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step()
        torch.cuda.synchronize()
    rows = [(e.key, e.device_time_total, e.count) for e in prof.key_averages() if e.device_time_total > 0]
    rows.sort(key=lambda r: -r[1])
    total = sum(r[1] for r in rows)
    print(f"layers={args.layers or 'all'} batch={args.batch} seq={args.seq}: {total / 1e3:.2f} ms of kernels in one step")
    print(f"{'share':>7} {'ms':>9} {'calls':>6}  kernel")
    for name, t, n in rows[: args.rows]:
        print(f"{100 * t / total:6.2f}% {t / 1e3:9.3f} {n:6d}  {name[:110]}")
    return rows


if __name__ == "__main__":
    main()
