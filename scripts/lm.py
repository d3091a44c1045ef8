"""Language-model pre-training entry point.

    torchrun --nproc-per-node N scripts/lm.py --conf <experiment config.py> [key=value ...]
        [--profile-steps a:b]     # steps a..b-1 under cudaProfilerStart/Stop + torch.profiler

Counterpart of the reference's scripts/lm.py; the loop itself lives in
`halite_b200.projects.lm.train.LMTrainer`.
"""

import sys

import torch.distributed as dist

from halite_b200.conf import load_arg_config
from halite_b200.projects.lm.config import LMConfig
from halite_b200.projects.lm.train import LMTrainer


def pop_profile_steps(argv):
    """Take `--profile-steps a:b` (or `--profile-steps=a:b`) out of argv; returns the window text."""
    for i, a in enumerate(argv):
        if a == "--profile-steps":
            window = argv[i + 1]
            del argv[i:i + 2]
            return window
        if a.startswith("--profile-steps="):
            del argv[i]
            return a.split("=", 1)[1]
    return None


def main():
    window = pop_profile_steps(sys.argv)
    conf = load_arg_config(LMConfig)
    LMTrainer(conf, profile_steps=window).run()


if __name__ == "__main__":
    main()
    if dist.is_initialized():
        dist.destroy_process_group()
