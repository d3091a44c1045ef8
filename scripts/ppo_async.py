"""Asynchronous, disaggregated PPO / GRPO entry point: trainer ranks and generator ranks in one
job, rollouts streamed through a replay buffer, weights pushed to the generators as training
proceeds (counterpart of the reference's scripts/ppo_monarch.py / ppo_monarch_rdma.py, which use
the Monarch actor runtime and RDMA buffers; here the roles are plain ranks, weights travel by an
NCCL broadcast).

    torchrun --nproc-per-node 8 scripts/ppo_async.py --conf configs/reasoning/math.py qwen3_0_6b_grpo \
        monarch.trainer_mesh_size=4 monarch.generator_mesh_size=4
"""

import torch.distributed as dist

from halite_b200.conf import load_arg_config
from halite_b200.projects.ppo.config import PPOConfig
from halite_b200.projects.ppo.train_async import AsyncPPOLoop


def main():
    conf = load_arg_config(PPOConfig)
    AsyncPPOLoop(conf).run()


if __name__ == "__main__":
    main()
    if dist.is_initialized():
        dist.destroy_process_group()
