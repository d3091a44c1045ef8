"""Language-model training runtime behind `scripts/lm.py` and `scripts/sft.py`
(reference behaviour: scripts/lm.py:26-437, scripts/sft.py:22-378).

Differences in mechanism: batches are staged through pinned host memory and copied to the
device on a side stream one step ahead; losses stay on the device and are only read at log
steps; the update itself is `optimization_step` (main-grad wgrad GEMMs, reduce-scatter
overlapped with backward, fused sharded AdamW with the clip coefficient read on the device);
checkpoints resume the loader position, optimizer and schedule.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from halite_b200.conf import instantiate, summarize
from halite_b200.data.dataloader import DataLoader, DataManager
from halite_b200.data.dataset import WeightedIterableDataset, build_dataset_from_spec
from halite_b200.distributed.checkpoint import CheckpointManager, load_checkpoint
from halite_b200.logging import get_logger
from halite_b200.optim import build_optimizer
from halite_b200.optim.sharded_adamw import clip_grad_norm_
from halite_b200.parallel import ParallelDims
from halite_b200.utils import nvtx
from halite_b200.utils.throughput import ThroughputMeter, model_flops_per_token

try:  # experiment tracking is optional
    import wandb
except ImportError:  # pragma: no cover
    wandb = None


class DevicePrefetcher:
    """Keeps one batch in flight: while step N computes, batch N+1 is pinned and copied
    host-to-device on its own stream. Iteration order and stop behaviour are the source's."""

    def __init__(self, source, device):
        self.source = iter(source)
        self.device = torch.device(device)
        self.stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self._next = None
        self._preload()

    def _preload(self):
        try:
            batch = next(self.source)
        except StopIteration:
            self._next = None
            return
        if self.stream is None:
            self._next = batch.to(self.device) if hasattr(batch, "to") else batch
            return
        if hasattr(batch, "pin_memory"):
            batch = batch.pin_memory()
        with torch.cuda.stream(self.stream):
            self._next = batch.to(self.device, non_blocking=True)

    def __iter__(self):
        return self

    def __next__(self):
        if self._next is None:
            raise StopIteration
        if self.stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
        batch = self._next
        if self.stream is not None:
            for v in batch.values():
                if isinstance(v, torch.Tensor) and v.is_cuda:
                    v.record_stream(torch.cuda.current_stream(self.device))
        self._preload()
        return batch


def _forward_loss(conf, model, criterion, batch, step_fn=None):
    if step_fn is not None:
        loss, loss_dict = step_fn(batch, model, criterion)
        return loss, dict(loss_dict)
    if conf.training.calc_loss_in_model:
        out = model(batch["input"], target=batch["target"])
        loss, loss_dict = out.loss, dict(out.loss_dict or {})
    else:
        out = model(batch["input"])
        loss, loss_dict = criterion(out.logits, batch["target"])
        loss_dict = dict(loss_dict)
    for aux in out.aux_outputs or []:
        if aux is None:
            continue
        for k, v in aux.items():
            loss_dict[k] = loss_dict.get(k, 0) + v.detach()
            loss = loss + v
    return loss, loss_dict


def _fmt(loss_dict):
    return "; ".join(f"{k}: {float(v):.5f}" for k, v in loss_dict.items() if k not in ("loss_vals", "n_targets"))


class LMTrainer:
    def __init__(self, conf, device=None, sft=False, num_workers=2, profile_steps=None):
        self.conf = conf
        self.sft = sft
        self.profile_steps = nvtx.parse_step_window(profile_steps) if isinstance(profile_steps, str) \
            else profile_steps
        t = conf.training
        self.pdims = ParallelDims(dp_replicate=t.data_parallel_replicate, dp_shard=t.data_parallel_shard,
                                  tp=t.tensor_parallel, pp=t.pipeline_parallel)
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device, self.pdims.local_rank) if device == "cuda" else torch.device(device)
        self.mesh = self.pdims.build_mesh(self.device.type)
        self.logger = get_logger(self.pdims)
        self.num_workers = num_workers
        self.global_step = 0
        torch.manual_seed(getattr(t, "seed", 42))

    # ------------------------------------------------------------------ construction
    def build_model(self):
        conf, log = self.conf, self.logger
        log.info("building model")
        with torch.device("meta"):
            model = instantiate(conf.model.model)
        for section in ("wrapper", "parallelize"):
            fn = getattr(conf.model, section, None)
            if fn is not None:
                log.info(f"applying {section}")
                kwargs = {"device": self.device} if self.device.type == "cpu" else {}
                model = instantiate(fn)(model=model, mesh=self.pdims, parallel_dims=self.pdims, **kwargs)
        if getattr(model, "_hb_fsdp", None) is None:
            model.to_empty(device=self.device)
        if conf.model.checkpoint_path is not None and self.sft:
            load_checkpoint(model, conf.model.checkpoint_path)
        else:
            model.init_weights(self.device)
        if conf.training.gradient_checkpointing:
            model.gradient_checkpointing_enable(1)
        self.model = model
        t = conf.training
        self.criterion = instantiate(t.criterion) if t.criterion is not None else None
        self.optimizer = build_optimizer(instantiate(t.optimizer), model, t.weight_decay)
        sched = instantiate(t.scheduler)
        self.scheduler = sched(optimizer=self.optimizer) if self.sft or t.max_iter is None \
            else sched(optimizer=self.optimizer, n_iter=t.max_iter)
        self.initializer = instantiate(t.model_initializer) if t.model_initializer is not None else None
        self.postprocess = instantiate(t.postprocess) if t.postprocess is not None else None
        self.train_step_fn = instantiate(t.train_step_fn) if t.train_step_fn is not None else None
        self.eval_step_fn = instantiate(t.eval_step_fn) if t.eval_step_fn is not None else self.train_step_fn
        return model

    def _dataset(self, spec, split, ratio, ops, shuffle=True):
        if spec is None:
            return None
        if not (isinstance(spec, dict) and "shards" in spec) and not hasattr(spec, "shards"):
            return instantiate(spec)          # an `Instance` that builds the dataset itself
        spec = spec if isinstance(spec, dict) else spec.model_dump()
        sources, ratios, names = build_dataset_from_spec(spec, split=split, split_ratio=ratio)
        return sources, ratios, names

    def build_data(self):
        conf, pd = self.conf, self.pdims
        ops = [instantiate(op) for op in (conf.data.preprocess or [])]
        ops_eval = [instantiate(op) for op in conf.data.preprocess_eval] if conf.data.preprocess_eval else ops
        collate = instantiate(conf.data.collate_fn) if conf.data.collate_fn is not None else None
        collate_eval = instantiate(conf.data.collate_fn_eval) if conf.data.collate_fn_eval is not None else collate
        dp, rank = pd.dp, pd.dp_rank
        train = self._dataset(conf.data.train, "train", conf.data.train_ratio, ops)
        if isinstance(train, tuple):
            train = WeightedIterableDataset(*train, num_replicas=dp, rank=rank, operations=ops,
                                            seed=getattr(conf.training, "seed", 42))
            self.logger.info(f"train_dset\n{train.summary()}")
        self.train_loader = DataLoader(train, batch_size=conf.training.train_batch_size // dp, collate_fn=collate,
                                       num_workers=self.num_workers, rank=rank, pin_memory=False)
        self.eval_loaders = []
        ev = self._dataset(conf.data.eval, "eval", conf.data.eval_ratio, ops_eval)
        if isinstance(ev, tuple):
            sources, ratios, names = ev
            groups = [(sources, ratios, names)] if self.sft else [([s], [1.0], [n]) for s, n in zip(sources, names)]
            for srcs, rts, nms in groups:
                d = WeightedIterableDataset(srcs, rts, nms, num_replicas=dp, rank=rank, operations=ops_eval,
                                            shuffle=False)
                self.eval_loaders.append(DataLoader(d, batch_size=conf.training.eval_batch_size // dp,
                                                    collate_fn=collate_eval, num_workers=0, rank=rank))
        elif ev is not None:
            self.eval_loaders.append(DataLoader(ev, batch_size=conf.training.eval_batch_size // dp,
                                                collate_fn=collate_eval, num_workers=0, rank=rank))

    def build_checkpointing(self):
        out = self.conf.output
        enabled = out.output_dir is not None and out.save_step is not None
        self.checkpoint = CheckpointManager(self.model, self.optimizer, self.scheduler, self.train_loader,
                                            model_config=self.conf.model, directory=out.output_dir or "checkpoint",
                                            interval=out.save_step or 0, enable_checkpoint=enabled)
        self.checkpoint.pre_save = self._check_kernels      # never write a state a timed-out kernel produced
        if enabled and self.checkpoint.load(-1):
            self.global_step = int(getattr(self.optimizer, "_step", 0))
            self.logger.info(f"resumed at step {self.global_step}")

    # ------------------------------------------------------------------ loops
    def _dp_group(self):
        return self.pdims.group("dp") if self.pdims.dp > 1 else None

    def _meter(self):
        return ThroughputMeter(None, self.pdims.dp, self.device)

    def _check_kernels(self):
        """Raise if a kernel of this process gave up a bounded wait (a peer that never signalled, a
        barrier that never completed): called where the loop reads from the device anyway."""
        if self.device.type == "cuda":
            from halite_b200 import ops

            ops.check_status(self.device)

    def train_epoch(self, epoch):
        conf, log, model = self.conf, self.logger, self.model
        model.train()
        if self.initializer is not None and self.global_step == 0:
            self.initializer(model)
        n_iter = len(self.train_loader)
        batches = DevicePrefetcher(DataManager(self.train_loader, self._dp_group(), device=self.device), self.device)
        step = 0
        fsdp = getattr(model, "_hb_fsdp", None)
        meter = self._meter()
        profiler = nvtx.StepWindowProfiler(self.profile_steps, conf.output.output_dir, log, self.pdims.rank)
        for batch in batches:
            profiler.step_begin(self.global_step)
            with nvtx.phase(f"step {self.global_step}"):
                with nvtx.phase("forward"):
                    loss, loss_dict = _forward_loss(conf, model, self.criterion, batch, self.train_step_fn)
                with nvtx.phase("backward"):
                    loss.backward()
                    loss = loss.detach()
                    if fsdp is not None:
                        fsdp.finish_backward()
                grad_norm = None
                with nvtx.phase("optimizer"):
                    if conf.training.clip_grad_norm is not None:
                        grad_norm = clip_grad_norm_(model, conf.training.clip_grad_norm, self.optimizer)
                    self.scheduler.step()
                    self.optimizer.step()
                    self.optimizer.zero_grad(set_to_none=True)
                    if self.postprocess is not None:
                        self.postprocess(model)
            profiler.step_end(self.global_step)
            inputs = batch["input"] if "input" in batch else None
            if isinstance(inputs, torch.Tensor):
                if meter.flops_per_token is None:
                    meter.flops_per_token = model_flops_per_token(model, inputs.shape[-1])
                meter.add(inputs.numel())
            if self.global_step % conf.output.log_step == 0:
                lr = self.optimizer.param_groups[0]["lr"]
                loss_val = float(loss)                     # the loop's one device -> host read
                self._check_kernels()
                speed = meter.lap()
                gn = "" if grad_norm is None else f" grad norm: {float(grad_norm):.3f};"
                sp = "" if not speed else (f" tokens/s: {speed['tokens_per_s']:.0f}; "
                                           f"mfu: {100 * speed.get('mfu', 0.0):.1f}%;")
                log.info(f"epoch {epoch}; {step}/{n_iter}; global {self.global_step}; loss: {loss_val:.5f}; "
                         f"{_fmt(loss_dict)};{gn}{sp} lr: {lr:.7f}")
                self.last_speed = speed or getattr(self, "last_speed", {})
                if self.pdims.is_primary and wandb is not None and wandb.run is not None:
                    report = {"train/loss": loss_val, "train/lr": lr}
                    report.update({f"train/{k}": float(v) for k, v in loss_dict.items()
                                   if k not in ("loss_vals",)})
                    report.update({f"perf/{k}": v for k, v in speed.items()})
                    if grad_norm is not None:
                        report["train/grad_norm"] = float(grad_norm)
                    wandb.log(report, step=self.global_step)
            self.global_step += 1
            step += 1
            if self.eval_loaders and step % conf.training.eval_step == 0:
                self.report_eval(self.evaluate())
            self.checkpoint.save(self.global_step)
            if conf.training.max_iter is not None and self.global_step >= conf.training.max_iter:
                break
        self.last_loss = float(loss) if step else None
        return step

    @torch.no_grad()
    def evaluate(self):
        """Mean of every loss entry over steps and ranks, plus the cross entropy per dataset
        (micro-averaged over target counts when the step function reports `n_targets`)."""
        conf, model = self.conf, self.model
        was_training = model.training
        model.eval()
        sums, per_set, per_set_n = {}, {}, {}
        weight_total, step = 0.0, 0
        total = sum(len(l) for l in self.eval_loaders)
        for batch in DevicePrefetcher(DataManager(self.eval_loaders, self._dp_group(), device=self.device),
                                      self.device):
            step += 1
            loss, loss_dict = _forward_loss(conf, model, self.criterion, batch, self.eval_step_fn)
            w = float(loss_dict.pop("n_targets", 1))
            weight_total += w
            for k, v in loss_dict.items():
                if k == "loss_vals":
                    continue
                v = v.float() * w if isinstance(v, torch.Tensor) else torch.tensor(float(v) * w, device=self.device)
                sums[k] = sums.get(k, 0) + v
            meta = getattr(batch, "_meta_", None) or batch.get("_meta_", None)
            name = None
            if meta and meta.get("samples_meta"):
                name = meta["samples_meta"][0].get("dataset_name")
            if name is not None and "cross entropy" in loss_dict:
                per_set[name] = per_set.get(name, 0.0) + float(loss_dict["cross entropy"])
                per_set_n[name] = per_set_n.get(name, 0) + 1
            if self.pdims.is_primary and step % conf.output.log_step == 0:
                self.logger.info(f"evaluating [{step}/{total}]; loss: {float(loss):.5f}")
        result = {}
        wt = torch.tensor([weight_total], dtype=torch.float32, device=self.device)
        group = self._dp_group()
        if group is not None:
            dist.all_reduce(wt, group=group)
        for k, v in sums.items():
            v = v.reshape(1).float()
            if group is not None:
                dist.all_reduce(v, group=group)
            result[k] = float(v / wt.clamp_min(1e-12))
        gathered = [(per_set, per_set_n)]
        if group is not None:
            gathered = [None] * self.pdims.dp
            dist.all_gather_object(gathered, (per_set, per_set_n), group=group)
        tot, cnt = {}, {}
        for s, n in gathered:
            for name, v in s.items():
                tot[name] = tot.get(name, 0.0) + v
                cnt[name] = cnt.get(name, 0) + n[name]
        for name in tot:
            result[f"loss/{name}"] = tot[name] / cnt[name]
        model.train(was_training)
        return result

    def report_eval(self, losses):
        self.logger.info(f"{_fmt(losses)} at step {self.global_step}")
        if self.pdims.is_primary and wandb is not None and wandb.run is not None:
            wandb.log({"eval/" + k: v for k, v in losses.items()}, step=self.global_step)

    # ------------------------------------------------------------------ entry
    def run(self):
        conf, log, pd = self.conf, self.logger, self.pdims
        log.info(summarize(conf))
        log.info(f"dp replicate: {pd.dp_replicate}, dp shard: {pd.dp_shard}, tp: {pd.tp} pp: {pd.pp}")
        if pd.is_primary and wandb is not None and conf.output.project is not None:
            name = conf.output.name
            if name is not None and not isinstance(name, str) and conf.hparams is not None:
                name = instantiate(name)(conf.hparams)
            wandb.init(project=conf.output.project, name=name, config=conf.hparams)
        if dist.is_initialized():
            dist.barrier()
        self.build_model()
        self.build_data()
        self.build_checkpointing()
        if self.eval_loaders and self.global_step == 0:
            log.info("evaluating baseline")
            self.report_eval(self.evaluate())
        log.info("start training")
        for epoch in range(conf.training.n_epochs):
            log.info(f"epoch {epoch}")
            self.train_epoch(epoch)
            if conf.training.max_iter is not None and self.global_step >= conf.training.max_iter:
                break
        if self.eval_loaders:
            log.info("final evaluation score")
            self.report_eval(self.evaluate())
        self.checkpoint.save(self.global_step, force=self.checkpoint.enable_checkpoint, last=True)
        self.checkpoint._wait() if self.checkpoint.enable_checkpoint else None
        return self
