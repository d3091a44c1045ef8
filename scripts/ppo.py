"""Synchronous colocated PPO / GRPO entry point (counterpart of the reference's scripts/ppo.py):
every rank trains the actor and, between updates, generates rollouts with the in-process paged
engine on the same GPU.

    torchrun --nproc-per-node N scripts/ppo.py --conf configs/reasoning/math.py [key=value ...]
"""

import torch.distributed as dist

from halite_b200.conf import load_arg_config
from halite_b200.projects.ppo.config import PPOConfig
from halite_b200.projects.ppo.train import PPOLoop


def main():
    conf = load_arg_config(PPOConfig)
    PPOLoop(conf).run()


if __name__ == "__main__":
    main()
    if dist.is_initialized():
        dist.destroy_process_group()
