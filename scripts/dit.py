"""Diffusion-transformer (JiT) training entry point (counterpart of the reference's scripts/dit.py).

    torchrun --nproc-per-node N scripts/dit.py --conf configs/exps/jit/jit.py [key=value ...]
"""

import torch.distributed as dist

from halite_b200.conf import load_arg_config
from halite_b200.projects.dit.config import DiTConfig
from halite_b200.projects.dit.train import DiTLoop


def main():
    conf = load_arg_config(DiTConfig)
    DiTLoop(conf).run()


if __name__ == "__main__":
    main()
    if dist.is_initialized():
        dist.destroy_process_group()
