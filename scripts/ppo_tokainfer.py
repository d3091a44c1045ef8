"""Synchronous colocated PPO / GRPO with the manager + worker generation engine (engine B):
same loop as scripts/ppo.py, rollouts scheduled several forwards ahead of the device
(counterpart of the reference's scripts/ppo_tokainfer.py).

    torchrun --nproc-per-node N scripts/ppo_tokainfer.py --conf configs/reasoning/math.py [key=value ...]
"""

import torch.distributed as dist

from halite_b200.conf import load_arg_config
from halite_b200.projects.ppo.config import PPOConfig
from halite_b200.projects.ppo.train import PPOLoop
from halite_b200.tokainfer import ServerConfig


def main():
    conf = load_arg_config(PPOConfig)
    server = ServerConfig(memory_fraction=conf.ppo.inference.memory_fraction)
    PPOLoop(conf, server_config=server, engine="tokainfer").run()


if __name__ == "__main__":
    main()
    if dist.is_initialized():
        dist.destroy_process_group()
