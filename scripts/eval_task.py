"""Generation-based evaluation of a saved model folder on one or more task configs
(counterpart of the reference's scripts/eval_task.py).

    torchrun --nproc-per-node N scripts/eval_task.py --model /path/to/model_dir \
        --task configs/eval/tasks/minerva_math/minerva_math.py [batch_size=16]
"""

import argparse
import json
import os

import torch
import torch.distributed as dist

from halite_b200.conf import load_config, summarize
from halite_b200.conf.loader import apply_overrides
from halite_b200.logging import get_logger
from halite_b200.parallel import ParallelDims
from halite_b200.projects.common.config import Model
from halite_b200.projects.eval.config import EvalTaskConfig, Task
from halite_b200.projects.eval.run import build_engine, run_task


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--task", action="append", required=True)
    ap.add_argument("--device", default=None)
    ap.add_argument("--max_batches", type=int, default=None)
    ap.add_argument("--output", default=None)
    ap.add_argument("opts", nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    tasks = []
    for path in args.task:
        for sub in load_config(path)["tasks"]:
            tasks.append(Task(**sub))
    eval_task = {}
    apply_overrides(eval_task, args.opts or [])
    return EvalTaskConfig(model=Model(checkpoint_path=args.model), tasks=tasks, eval_task=eval_task), args


def main(argv=None):
    conf, args = parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    pdims = ParallelDims(dp_replicate=world, dp_shard=1)
    device = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    pdims.build_mesh(device)
    logger = get_logger(pdims)
    logger.info(summarize(conf))
    engine = build_engine(conf.model, device=torch.device(device, pdims.local_rank) if device == "cuda" else device)
    results = {}
    for task in conf.tasks:
        results[task.name] = run_task(engine, task, conf.eval_task, logger, pdims.rank, world, args.max_batches)
        logger.info(f"{task.name}: {json.dumps(results[task.name])}")
    if args.output and pdims.is_primary:
        with open(args.output, "w") as f:
            json.dump(results, f, indent=2)
    return results


if __name__ == "__main__":
    main()
    if dist.is_initialized():
        dist.destroy_process_group()
