"""Language-model pre-training entry point.

    torchrun --nproc-per-node N scripts/lm.py --conf <experiment config.py> [key=value ...]

Counterpart of the reference's scripts/lm.py; the loop itself lives in
`halite_b200.projects.lm.train.LMTrainer`.
"""

import torch.distributed as dist

from halite_b200.conf import load_arg_config
from halite_b200.projects.lm.config import LMConfig
from halite_b200.projects.lm.train import LMTrainer


def main():
    conf = load_arg_config(LMConfig)
    LMTrainer(conf).run()


if __name__ == "__main__":
    main()
    if dist.is_initialized():
        dist.destroy_process_group()
