"""Synchronous, colocated PPO / GRPO loop behind `scripts/ppo.py`
(reference behaviour: scripts/ppo.py:70-443).

Per step: take the device back for generation (`rollout_generator.initialize()`), hand the
engine the live actor weights, generate n samples per prompt, score them, release the KV pools,
compute advantages, then run `ppo_n_epochs` passes of minibatch / microbatch actor updates.

Mechanism differences: weights reach the engine by aliasing the trainer's resident bf16
parameters (no gather, no copy) whenever layouts agree; gradient clipping and AdamW are the fused
sharded kernels; metrics stay on the device until a log step.
"""

from __future__ import annotations

import contextlib

import gc

import torch
import torch.distributed as dist

from halite_b200.conf import instantiate, summarize
from halite_b200.data.dataloader import DataLoader, DataManager
from halite_b200.data.dataset import WeightedIterableDataset, build_dataset_from_spec
from halite_b200.distributed.checkpoint import CheckpointManager, load_checkpoint
from halite_b200.infer.engine import InferenceEngine
from halite_b200.infer.types import ModelConfig
from halite_b200.logging import get_logger
from halite_b200.optim import build_optimizer
from halite_b200.optim.sharded_adamw import clip_grad_norm_
from halite_b200.parallel import ParallelDims
from halite_b200.utils import get_torch_dtype

try:
    import wandb
except ImportError:  # pragma: no cover
    wandb = None


def clean_memory():
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def build_rollout_report(conf, rollouts):
    """A few (input, output, reward) samples as text for the log."""
    texts, shown = [], 0
    for i, r in enumerate(rollouts.rollouts):
        if i % conf.show_every_nth_sample:
            continue
        reward = r.rewards_dict[conf.reward_key]
        reward = reward.to("cpu") if hasattr(reward, "to") else reward
        text = f"# {i}\n[input]\n{r.get_field(conf.input_key)}\n\n[output]\n{r.get_field(conf.output_key)}\n\n[reward]\n{reward}"
        for key in conf.additional_keys or []:
            text += f"\n\n[{key}]\n{r.get_field(key)}"
        texts.append(text)
        shown += 1
        if shown >= conf.show_n_samples:
            break
    return "\n\n".join(texts)


def _get(conf, key, default=None):
    if conf is None:
        return default
    if hasattr(conf, "get"):
        return conf.get(key, default)
    return getattr(conf, key, default)


class PPOLoop:
    def __init__(self, conf, device=None, server_config=None, num_workers=4, engine="paged"):
        """`engine`: "paged" = the in-process engine, "tokainfer" = the manager + worker engine."""
        self.conf = conf
        self.engine_kind = engine
        t = conf.training
        self.pdims = ParallelDims(dp_replicate=t.data_parallel_replicate, dp_shard=t.data_parallel_shard,
                                  tp=t.tensor_parallel, pp=t.pipeline_parallel)
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device, self.pdims.local_rank) if device == "cuda" else torch.device(device)
        self.pdims.build_mesh(self.device.type)
        self.logger = get_logger(self.pdims)
        self.server_config = server_config
        self.num_workers = num_workers
        self.global_step = 0
        self.history = []

    # ------------------------------------------------------------------ construction
    def build_model(self, conf, kind="model"):
        self.logger.info(f"building the {kind}")
        with torch.device("meta"):
            model = instantiate(conf.model)
        dtype = _get(conf.model_conf, "dtype", None)
        wrapped = False
        for section in ("wrapper", "parallelize"):
            fn = getattr(conf, section, None)
            if fn is not None:
                kwargs = {"device": self.device} if self.device.type == "cpu" else {}
                model = instantiate(fn)(model=model, mesh=self.pdims, parallel_dims=self.pdims, **kwargs)
                wrapped = True
        if getattr(model, "_hb_fsdp", None) is None:
            model.to_empty(device=self.device)
            if dtype is not None and not wrapped:
                model.to(get_torch_dtype(dtype))
        if conf.checkpoint_path is not None:
            load_checkpoint(model, conf.checkpoint_path)
        else:
            model.init_weights(self.device)
        return model

    def build(self):
        self.build_training()
        self.build_generation()
        self.build_data()
        self.build_optimizer()
        return self

    def build_training(self):
        conf, ppo = self.conf, self.conf.ppo
        self.actor = self.build_model(ppo.actor, "actor")
        self.ref = self.build_model(ppo.ref, "reference policy") if ppo.ref is not None else None
        self.critic = self.build_model(ppo.critic, "critic") if ppo.critic is not None else None
        if self.ref is not None:
            self.ref.requires_grad_(False)
        actor_train = instantiate(ppo.actor_wrapper)(self.actor) if ppo.actor_wrapper is not None else self.actor
        self.trainer = instantiate(ppo.trainer)(actor=actor_train, ref=self.ref, critic=self.critic, device=self.device)

    def build_generation(self):
        conf, ppo = self.conf, self.conf.ppo
        # generation side: the same architecture rewritten for the paged engine
        with torch.device("meta"):
            infer_conf = instantiate(ppo.actor.model_infer)
            if callable(infer_conf) and not isinstance(infer_conf, torch.nn.Module):
                infer_conf = instantiate(infer_conf(ppo.actor.model))
            actor_infer = infer_conf
        if ppo.actor.parallelize_infer is not None:
            actor_infer = instantiate(ppo.actor.parallelize_infer)(model=actor_infer, mesh=self.pdims,
                                                                   parallel_dims=self.pdims)
        infer_dtype = get_torch_dtype(ppo.infer_dtype) if self.device.type == "cuda" else torch.float32
        actor_infer = actor_infer.to(dtype=infer_dtype)
        actor_infer.to_empty(device=self.device)
        self.tokenizer = instantiate(ppo.actor.tokenizer)
        mc = ppo.actor.model_conf
        engine_cls = InferenceEngine
        if self.engine_kind == "tokainfer":
            from halite_b200.tokainfer import InferenceEngine as engine_cls
        self.engine = engine_cls(
            actor_infer, self.tokenizer,
            ModelConfig(n_heads=_get(mc, "n_heads"), n_key_value_heads=_get(mc, "n_key_value_heads") or _get(mc, "n_heads"),
                        head_dim=_get(mc, "head_dim"), n_layers=_get(mc, "n_layers"), context_len=_get(mc, "context_len"),
                        memory_fraction_static=ppo.inference.memory_fraction, kv_cache_dtype=infer_dtype,
                        gpu_id=self.pdims.local_rank, device=self.device.type, distributed=dist.is_initialized(),
                        vocab_size=_get(mc, "vocab_size")),
            self.server_config)
        self.request_builder = instantiate(ppo.request_builder)
        self.rollout_generator = instantiate(ppo.rollout_generator)(self.engine)

    def build_data(self):
        conf = self.conf
        ops = [instantiate(op) for op in (conf.data.preprocess or [])]
        collate = instantiate(conf.data.collate_fn) if conf.data.collate_fn is not None else None
        dp, rank = self.pdims.dp, self.pdims.dp_rank
        spec = conf.data.train
        if hasattr(spec, "model_dump") or (isinstance(spec, dict) and "shards" in spec):
            spec = spec if isinstance(spec, dict) else spec.model_dump()
            train = WeightedIterableDataset(*build_dataset_from_spec(spec, "train", conf.data.train_ratio),
                                            num_replicas=dp, rank=rank, operations=ops)
            self.logger.info(f"train_dset\n{train.summary()}")
        else:
            train = instantiate(spec)
        self.train_loader = DataLoader(train, batch_size=conf.training.train_batch_size // dp, collate_fn=collate,
                                       num_workers=self.num_workers, rank=rank, drop_last=True)

    def build_optimizer(self):
        conf, ppo = self.conf, self.conf.ppo
        t = conf.training
        self.optimizer = build_optimizer(instantiate(t.optimizer), self.actor, t.weight_decay)
        self.scheduler = instantiate(t.scheduler)(optimizer=self.optimizer)
        out = conf.output
        enabled = out.output_dir is not None and out.save_step is not None
        self.checkpoint = CheckpointManager(self.actor, self.optimizer, self.scheduler, self.train_loader,
                                            model_config=ppo.actor, directory=out.output_dir or "checkpoint",
                                            interval=out.save_step or 0, enable_checkpoint=enabled)
        if enabled and self.checkpoint.load(-1):
            self.global_step = int(getattr(self.optimizer, "_step", 0))
        return self

    # ------------------------------------------------------------------ one iteration
    def generate(self, batch):
        clean_memory()
        gen = self.rollout_generator
        gen.initialize()
        gen.load_from_model(self.actor)
        rollout = gen.generate(self.request_builder(batch))
        gen.cleanup()
        clean_memory()
        return rollout

    def update(self, rollout):
        """Advantages, then the minibatch / microbatch actor updates. Returns (metrics, grad_norm)."""
        t = self.conf.training
        rollout = self.trainer.compute_advantage(rollout)
        minibatches = rollout.split(t.ppo_minibatch_size) if t.ppo_minibatch_size is not None else [rollout]
        metrics, grad_norm, n_micro = [], None, 1
        fsdp = getattr(self.actor, "_hb_fsdp", None)
        self.scheduler.step()
        for _ in range(t.ppo_n_epochs):
            for mb in minibatches:
                self.optimizer.zero_grad(set_to_none=True)
                micro = mb.split(t.ppo_microbatch_size) if t.ppo_microbatch_size is not None else [mb]
                n_micro = len(micro)
                for i, m in enumerate(micro):
                    # only the last micro-batch's backward starts the gradient reductions
                    hold = fsdp.no_sync() if fsdp is not None and i < n_micro - 1 else contextlib.nullcontext()
                    with hold:
                        res = self.trainer.compute_actor_loss(m)
                        (res.loss / n_micro).backward()
                    d = {k: (v.detach() if isinstance(v, torch.Tensor) else v) for k, v in res.metric_dict().items()}
                    d["sample/response_len/mean"] = m.batch.response_len.float().mean()
                    metrics.append(d)
                if fsdp is not None:
                    fsdp.finish_backward()
                if t.clip_grad_norm is not None:
                    grad_norm = clip_grad_norm_(self.actor, t.clip_grad_norm, self.optimizer)
                self.optimizer.step()
        self.n_minibatches, self.n_microbatches = len(minibatches), n_micro
        if self.device.type == "cuda":
            from halite_b200 import ops

            # `reduce_metrics` reads from the device right after this: a kernel that gave up a
            # bounded wait during the update raises here instead of training on
            ops.check_status(self.device)
        return rollout, metrics, grad_norm

    def reduce_metrics(self, metrics):
        acc = {}
        for m in metrics:
            for k, v in m.items():
                acc.setdefault(k, []).append(torch.as_tensor(v, dtype=torch.float32, device=self.device))
        keys = sorted(acc)
        if not keys:
            return {}
        flat = torch.stack([torch.stack(acc[k]).mean() for k in keys])
        group = self.pdims.group("dp") if self.pdims.dp > 1 else None
        if group is not None:
            dist.all_reduce(flat, group=group)
            flat = flat / self.pdims.dp
        return dict(zip(keys, flat.tolist()))            # one device -> host read for all metrics

    def train_epoch(self, epoch):
        conf, log = self.conf, self.logger
        group = self.pdims.group("dp") if self.pdims.dp > 1 else None
        n_iter = len(self.train_loader)
        step = 0
        for batch in DataManager(self.train_loader, group, device=self.device):
            batch = batch.to(self.device)
            rollout = self.generate(batch)
            rollout, metrics, grad_norm = self.update(rollout)
            if self.global_step == 0:
                log.info(f"ppo epochs: {conf.training.ppo_n_epochs}, minibatches: {self.n_minibatches}, "
                         f"microbatches: {self.n_microbatches}")
            report = conf.ppo.report
            if report is not None and self.global_step % report.log_step == 0:
                log.info(build_rollout_report(report, rollout))
            if self.global_step % min(conf.output.log_step, conf.output.wandb_log_step) == 0:
                mean = self.reduce_metrics(metrics)
                self.history.append((self.global_step, mean))
                lr = self.optimizer.param_groups[0]["lr"]
                txt = "; ".join(f"{k}: {v:.5f}" for k, v in mean.items())
                gn = "" if grad_norm is None else f" grad norm: {float(grad_norm):.3f};"
                if self.global_step % conf.output.log_step == 0:
                    log.info(f"epoch {epoch}; {step}/{n_iter}; global {self.global_step}; {txt};{gn} lr: {lr:.7f}")
                if self.pdims.is_primary and wandb is not None and wandb.run is not None and \
                        self.global_step % conf.output.wandb_log_step == 0:
                    wandb.log({"actor/lr": lr, **mean, **({"actor/grad_norm": float(grad_norm)} if grad_norm is not None else {})},
                              step=self.global_step)
            self.global_step += 1
            step += 1
            self.checkpoint.save(self.global_step)
            if conf.training.max_iter is not None and self.global_step >= conf.training.max_iter:
                break
        return step

    def run(self):
        conf, log, pd = self.conf, self.logger, self.pdims
        log.info(summarize(conf))
        log.info(f"dp replicate: {pd.dp_replicate}, dp shard: {pd.dp_shard}, tp: {pd.tp} pp: {pd.pp}")
        if pd.is_primary and wandb is not None and conf.output.project is not None:
            wandb.init(project=conf.output.project, name=conf.output.name if isinstance(conf.output.name, str) else None)
        if dist.is_initialized():
            dist.barrier()
        self.build()
        for epoch in range(conf.training.n_epochs):
            log.info(f"epoch {epoch}")
            self.train_epoch(epoch)
            if conf.training.max_iter is not None and self.global_step >= conf.training.max_iter:
                break
        if self.checkpoint.enable_checkpoint:
            self.checkpoint._wait()
        return self
