"""Supervised fine-tuning entry point: starts from `model.checkpoint_path`, uses the configured
`train_step_fn` / `eval_step_fn`, evaluates one mixed eval set and checkpoints every
`output.save_step` steps (counterpart of the reference's scripts/sft.py).

    torchrun --nproc-per-node N scripts/sft.py --conf <experiment config.py> [key=value ...]
"""

import os
import sys

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from halite_b200.conf import load_arg_config
from halite_b200.projects.lm.config import LMConfig
from halite_b200.projects.lm.train import LMTrainer


def main():
    from scripts.lm import pop_profile_steps

    window = pop_profile_steps(sys.argv)
    conf = load_arg_config(LMConfig)
    LMTrainer(conf, sft=True, num_workers=4, profile_steps=window).run()


if __name__ == "__main__":
    main()
    if dist.is_initialized():
        dist.destroy_process_group()
