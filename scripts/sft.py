"""Supervised fine-tuning entry point: starts from `model.checkpoint_path`, uses the configured
`train_step_fn` / `eval_step_fn`, evaluates one mixed eval set and checkpoints every
`output.save_step` steps (counterpart of the reference's scripts/sft.py).

    torchrun --nproc-per-node N scripts/sft.py --conf <experiment config.py> [key=value ...]
"""

import torch.distributed as dist

from halite_b200.conf import load_arg_config
from halite_b200.projects.lm.config import LMConfig
from halite_b200.projects.lm.train import LMTrainer


def main():
    conf = load_arg_config(LMConfig)
    LMTrainer(conf, sft=True, num_workers=4).run()


if __name__ == "__main__":
    main()
    if dist.is_initialized():
        dist.destroy_process_group()
