"""Diffusion-transformer training loop behind `scripts/dit.py` (reference: scripts/dit.py:25-306):
flow-matching loss, EMA of the weights, periodic class-conditional sampling from the EMA model,
EMA checkpoints.

The EMA of a sharded model lives on the flat fp32 master shards (one `lerp_` per unit per step,
no per-parameter loop); sampling swaps the EMA shards in, re-gathers, generates, and swaps back.
"""

from __future__ import annotations

import contextlib
import os

import numpy as np
import torch
import torch.distributed as dist
from torch.utils.data import DataLoader, DistributedSampler

from halite_b200.conf import instantiate, summarize
from halite_b200.distributed.checkpoint import load_checkpoint
from halite_b200.logging import get_logger
from halite_b200.optim import build_optimizer
from halite_b200.parallel import ParallelDims

try:
    import wandb
except ImportError:  # pragma: no cover
    wandb = None


class EMA:
    def __init__(self, model, decay):
        self.model, self.decay = model, decay
        self.fsdp = getattr(model, "_hb_fsdp", None)
        if self.fsdp is not None:
            self.shadow = [u.master.clone() for u in self.fsdp.units]
        else:
            self.shadow = {n: p.detach().clone().float() for n, p in model.named_parameters() if p.requires_grad}

    @torch.no_grad()
    def update(self):
        w = 1 - self.decay
        if self.fsdp is not None:
            for s, u in zip(self.shadow, self.fsdp.units):
                s.lerp_(u.master, w)
        else:
            for n, p in self.model.named_parameters():
                if n in self.shadow:
                    self.shadow[n].lerp_(p.detach().float(), w)

    @contextlib.contextmanager
    def applied(self):
        """Run a block with the averaged weights loaded into the live model."""
        with torch.no_grad():
            if self.fsdp is not None:
                saved = [u.master.clone() for u in self.fsdp.units]
                for s, u in zip(self.shadow, self.fsdp.units):
                    u.master.copy_(s)
                    u.param_shard().copy_(s)
                    u.start_gather()
                for u in self.fsdp.units:
                    u.wait_gather()
            else:
                saved = {n: p.detach().clone() for n, p in self.model.named_parameters() if n in self.shadow}
                for n, p in self.model.named_parameters():
                    if n in self.shadow:
                        p.copy_(self.shadow[n])
        try:
            yield self.model
        finally:
            with torch.no_grad():
                if self.fsdp is not None:
                    for s, u in zip(saved, self.fsdp.units):
                        u.master.copy_(s)
                        u.param_shard().copy_(s)
                        u.start_gather()
                    for u in self.fsdp.units:
                        u.wait_gather()
                else:
                    for n, p in self.model.named_parameters():
                        if n in saved:
                            p.copy_(saved[n])

    def state_dict(self):
        """Full (unsharded) averaged weights keyed like the model."""
        with self.applied() as m:
            return {k: v.detach().to("cpu").clone() for k, v in m.state_dict().items()}


def make_grid(images, nrow):
    """[N, C, H, W] in [0, 1] -> one [C, rows*H, nrow*W] uint8 image."""
    n, c, h, w = images.shape
    rows = (n + nrow - 1) // nrow
    canvas = images.new_zeros(c, rows * h, nrow * w)
    for i in range(n):
        r, col = divmod(i, nrow)
        canvas[:, r * h:(r + 1) * h, col * w:(col + 1) * w] = images[i]
    return (canvas.clamp(0, 1) * 255).to("cpu", torch.uint8)


class DiTLoop:
    def __init__(self, conf, device=None, num_workers=8):
        self.conf = conf
        t = conf.training
        self.pdims = ParallelDims(dp_replicate=t.data_parallel_replicate, dp_shard=t.data_parallel_shard,
                                  tp=t.tensor_parallel, pp=t.pipeline_parallel)
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device, self.pdims.local_rank) if device == "cuda" else torch.device(device)
        self.pdims.build_mesh(self.device.type)
        self.logger = get_logger(self.pdims)
        self.num_workers = num_workers
        self.global_step = 0
        self.losses = []
        seed = t.seed + self.pdims.rank
        torch.manual_seed(seed)
        np.random.seed(seed)

    def build_model(self):
        mc = self.conf.model
        with torch.device("meta"):
            model = instantiate(mc.model)
        if mc.wrapper is not None:
            model = instantiate(mc.wrapper)(model)
        if mc.parallelize is not None:
            kwargs = {"device": self.device} if self.device.type == "cpu" else {}
            model = instantiate(mc.parallelize)(model=model, mesh=self.pdims, parallel_dims=self.pdims, **kwargs)
        if getattr(model, "_hb_fsdp", None) is None:
            model.to_empty(device=self.device)
        model.init_weights(self.device)
        if mc.checkpoint_path is not None:
            load_checkpoint(model, mc.checkpoint_path)
        fsdp = getattr(model, "_hb_fsdp", None)
        if fsdp is not None:                   # initialisation wrote the parameters: refresh shards
            fsdp.sync_parameters()
        return model

    def build(self):
        conf, t = self.conf, self.conf.training
        self.model = self.build_model()
        if t.freeze_encoder and hasattr(self.model, "freeze_encoder"):
            self.model.freeze_encoder()
        self.criterion = instantiate(t.criterion)
        self.optimizer = build_optimizer(instantiate(t.optimizer), self.model, t.weight_decay)
        self.ema = EMA(self.model, t.ema)
        dset = instantiate(conf.data.train)
        dp, rank = self.pdims.dp, self.pdims.dp_rank
        self.sampler = DistributedSampler(dset, num_replicas=dp, rank=rank, shuffle=True, seed=t.seed)
        self.loader = DataLoader(dset, sampler=self.sampler, batch_size=t.train_batch_size // dp,
                                 num_workers=self.num_workers, drop_last=True, pin_memory=self.device.type == "cuda")
        per_epoch = len(self.loader)
        sched = instantiate(t.scheduler)
        warm = sched.keywords.get("warmup", 0) if hasattr(sched, "keywords") else 0
        self.scheduler = sched(optimizer=self.optimizer, warmup=int(warm * per_epoch), n_iter=t.n_epochs * per_epoch)
        out = conf.output
        self.output_path = None
        if out.output_dir is not None:
            name = out.name if isinstance(out.name, str) else "run"
            self.output_path = os.path.join(out.output_dir, name)
            if self.pdims.is_primary:
                os.makedirs(self.output_path, exist_ok=True)
        return self

    def _group(self):
        return self.pdims.group("dp") if self.pdims.dp > 1 else None

    @torch.no_grad()
    def sample(self):
        """Class-conditional samples from the EMA weights, gathered over ranks into a grid."""
        t = self.conf.training
        per_rank = max(1, t.eval_batch_size // self.pdims.dp)
        r = self.pdims.dp_rank
        labels = torch.arange(r * per_rank, (r + 1) * per_rank, device=self.device) % self.criterion.n_labels
        with self.ema.applied() as model:
            was = model.training
            model.eval()
            samples = self.criterion.generate(model, labels, seed=t.seed)
            model.train(was)
        samples = ((samples + 1) / 2).clamp(0, 1)
        group = self._group()
        if group is not None:
            full = samples.new_zeros(per_rank * self.pdims.dp, *samples.shape[1:])
            dist.all_gather_into_tensor(full, samples.contiguous(), group=group)
            samples = full
        grid = make_grid(samples, max(1, round(samples.shape[0] ** 0.5)))
        if self.pdims.is_primary and self.output_path is not None:
            path = os.path.join(self.output_path, f"samples-{self.global_step:07d}")
            try:
                from PIL import Image

                Image.fromarray(grid.permute(1, 2, 0).numpy()).save(path + ".png")
            except ImportError:
                torch.save(grid, path + ".pt")
        if self.pdims.is_primary and wandb is not None and wandb.run is not None:
            wandb.log({"samples": wandb.Image(grid)}, step=self.global_step)
        return grid

    def save_ema(self):
        sd = self.ema.state_dict()
        if self.pdims.is_primary and self.output_path is not None:
            torch.save(sd, os.path.join(self.output_path, f"ema-{self.global_step:07d}.pt"))

    def train_epoch(self, epoch):
        conf, log = self.conf, self.logger
        self.model.train()
        self.criterion.train()
        n_iter = len(self.loader)
        fsdp = getattr(self.model, "_hb_fsdp", None)
        step = 0
        for step, (images, labels) in enumerate(self.loader):
            images = images.to(self.device, non_blocking=True).float().div_(255).mul_(2).sub_(1)
            labels = labels.to(self.device, non_blocking=True).long()
            loss = self.criterion.loss(self.model, images, labels)
            self.optimizer.zero_grad(set_to_none=True)
            loss.backward()
            if fsdp is not None:
                fsdp.finish_backward()
            self.scheduler.step()
            self.optimizer.step()
            self.ema.update()
            if step % conf.output.log_step == 0:
                val = loss.detach().float().clone()
                if self._group() is not None:
                    dist.all_reduce(val, group=self._group())
                    val /= self.pdims.dp
                lr = self.optimizer.param_groups[0]["lr"]
                self.losses.append(val.item())
                if self.device.type == "cuda":
                    from halite_b200 import ops

                    ops.check_status(self.device)       # a bounded wait that ran out raises here
                log.info(f"epoch {epoch}; {step}/{n_iter}; global {self.global_step}; loss: {val.item():.5f}; lr: {lr:.7f}")
                if self.pdims.is_primary and wandb is not None and wandb.run is not None:
                    wandb.log({"train/loss": val.item(), "train/lr": lr}, step=self.global_step)
            if self.global_step % conf.output.sampling_step == 0:
                self.sample()
            if conf.output.save_step and self.global_step % conf.output.save_step == 0:
                self.save_ema()
            self.global_step += 1
            if conf.training.max_iter is not None and self.global_step >= conf.training.max_iter:
                break
        return step + 1

    def run(self):
        conf, log, pd = self.conf, self.logger, self.pdims
        log.info(summarize(conf))
        log.info(f"dp replicate: {pd.dp_replicate}, dp shard: {pd.dp_shard}, tp: {pd.tp} pp: {pd.pp}")
        if pd.is_primary and wandb is not None and conf.output.project is not None:
            wandb.init(project=conf.output.project, name=conf.output.name if isinstance(conf.output.name, str) else None,
                       config=conf.hparams)
        if dist.is_initialized():
            dist.barrier()
        self.build()
        log.info("start training")
        for epoch in range(conf.training.n_epochs):
            self.sampler.set_epoch(epoch)
            self.train_epoch(epoch)
            if conf.training.max_iter is not None and self.global_step >= conf.training.max_iter:
                break
        self.save_ema()
        return self
