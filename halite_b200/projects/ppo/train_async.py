"""Asynchronous, disaggregated PPO / GRPO (reference: scripts/ppo_monarch.py:167-731).

One job, two roles. Ranks [0, T) train the actor (their own `torch.distributed` world of size
T); ranks [T, T + G) only generate, each with its own paged engine. Trainer 0 runs the rollout
manager: it streams prompt batches to the generators and collects scored rollouts in a replay
buffer. Training consumes the buffer as rollouts arrive, so generation of the next batches
overlaps with the update; every `sync_interval` updates the new weights are pushed to the
generators, which pick them up between engine calls. Rollouts older than `max_staleness` policy
versions are dropped.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from halite_b200.distributed.process_group import PyNcclCommunicator, StatelessProcessGroup
from halite_b200.projects.common.rollout_async import (GeneratorWorker, ReplayBuffer, RolloutManager, TensorSpec,
                                                       WeightChannel, chunk_list)
from halite_b200.projects.ppo.train import PPOLoop


def split_roles(conf):
    """(n_trainers, n_generators, rank, role) from the job's environment and the `monarch` section."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    m = conf.monarch
    n_gen = m.generator_mesh_size if m is not None else 1
    n_train = m.trainer_mesh_size if m is not None else world - n_gen
    if n_train + n_gen != world:
        raise ValueError(f"trainer ({n_train}) + generator ({n_gen}) ranks must equal the world size ({world})")
    return n_train, n_gen, rank, ("trainer" if rank < n_train else "generator")


class AsyncPPOLoop(PPOLoop):
    def __init__(self, conf, device=None, server_config=None, num_workers=0, sync_interval=1, max_staleness=1,
                 engine="paged"):
        self.n_train, self.n_gen, self.job_rank, self.role = split_roles(conf)
        self.job_world = self.n_train + self.n_gen
        self.base_port = int(os.environ.get("MASTER_PORT", "29500"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        # trainers form their own torch.distributed world; generators never join one
        os.environ["MASTER_PORT"] = str(self.base_port + 1)
        if self.role == "trainer":
            os.environ["WORLD_SIZE"], os.environ["RANK"] = str(self.n_train), str(self.job_rank)
        else:
            os.environ["WORLD_SIZE"], os.environ["RANK"] = "1", "0"
        conf.training.data_parallel_shard = self.n_train if self.role == "trainer" else 1
        conf.training.data_parallel_replicate = 1
        super().__init__(conf, device, server_config, num_workers, engine)
        if self.device.type == "cuda":
            self.device = torch.device("cuda", self.local_rank)
            torch.cuda.set_device(self.device)
        self.sync_interval, self.max_staleness = sync_interval, max_staleness
        self.control = StatelessProcessGroup.create(os.environ.get("MASTER_ADDR", "127.0.0.1"), self.base_port + 2,
                                                    self.job_rank, self.job_world)
        self.generator_ranks = list(range(self.n_train, self.job_world))
        comm = None
        if self.device.type == "cuda" and (self.job_rank == 0 or self.role == "generator"):
            # NCCL communicator over {trainer 0} + generators for weight broadcast
            sub = StatelessProcessGroup.create(os.environ.get("MASTER_ADDR", "127.0.0.1"), self.base_port + 3,
                                               0 if self.job_rank == 0 else self.job_rank - self.n_train + 1,
                                               self.n_gen + 1)
            comm = PyNcclCommunicator(sub, self.device)
        self.weights = WeightChannel(self.control, 0, self.generator_ranks, comm)

    # ------------------------------------------------------------------ generator role
    def run_generator(self):
        self.build_generation()
        worker = GeneratorWorker(self.control, self.job_rank, 0, self.engine, self.rollout_generator,
                                 self.request_builder, self.weights, self.device)
        worker.run()
        return worker

    # ------------------------------------------------------------------ trainer role
    def _push_weights(self, version):
        sd = {k: v.detach() for k, v in self.actor.state_dict().items()}
        if self.weights.comm is None:
            payload = {k: v.to("cpu").clone() for k, v in sd.items()}
            specs = [TensorSpec.from_tensor(k, v) for k, v in payload.items()]
            self.manager.queue_weights(lambda g: self.control.send_obj(("weights", version, specs, payload), g))
        else:
            specs = [TensorSpec.from_tensor(k, v) for k, v in sd.items()]
            self.manager.queue_weights(lambda g: self.control.send_obj(("weights", version, specs, None), g))
            for v in sd.values():
                self.weights.comm.broadcast(v.contiguous(), src=0)

    def run_trainer(self):
        conf, log = self.conf, self.logger
        self.build_training()
        self.build_data()
        self.build_optimizer()
        group = self.pdims.group("dp") if self.pdims.dp > 1 else None
        if self.job_rank == 0:
            self.buffer = ReplayBuffer(capacity=4 * self.n_gen, max_staleness=self.max_staleness)

            def prompts():
                # the rollout manager consumes whole global batches: rank 0 reads every rank's share
                from halite_b200.data.dataloader import DataLoader

                loader = DataLoader(self.train_loader.dataset, batch_size=conf.training.train_batch_size // max(self.n_gen, 1),
                                    collate_fn=self.train_loader.collate_fn, num_workers=0, rank=0, drop_last=True)
                for _ in range(conf.training.n_epochs):
                    yield from loader

            self.manager = RolloutManager(self.control, self.generator_ranks, prompts(), self.buffer)
            self._push_weights(0)
            self.manager.start()
        max_iter = conf.training.max_iter or 1 << 30
        while self.global_step < max_iter:
            if self.job_rank == 0:
                try:
                    version, rollouts = self.buffer.get(self.global_step, timeout=600)
                    parts = chunk_list(rollouts, self.n_train)
                except TimeoutError:
                    version, parts = -1, None
            else:
                version, parts = None, None
            if group is not None:
                box = [(version, parts)]
                dist.broadcast_object_list(box, src=0, group=group)
                version, parts = box[0]
            if parts is None:
                break
            mine = parts[self.job_rank]
            rollout, metrics, grad_norm = self.update(mine)
            mean = self.reduce_metrics(metrics)
            self.history.append((self.global_step, mean))
            if self.global_step % conf.output.log_step == 0:
                txt = "; ".join(f"{k}: {v:.5f}" for k, v in mean.items())
                log.info(f"global {self.global_step}; policy version of rollouts {version}; {txt}")
            self.global_step += 1
            if self.job_rank == 0 and self.global_step % self.sync_interval == 0:
                self._push_weights(self.global_step)
            self.checkpoint.save(self.global_step)
        if self.job_rank == 0:
            self.manager.stop()
            log.info(f"replay buffer dropped {self.buffer.dropped} stale group(s)")
        return self

    def run(self):
        out = self.run_trainer() if self.role == "trainer" else self.run_generator()
        try:
            self.control.barrier(timeout=120)
        except RuntimeError:
            pass
        return out
