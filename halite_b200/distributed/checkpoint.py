"""Checkpoint save / load / resume (reference: distributed/checkpoint.py:78-388).

Layout: `<directory>/step-N/` is a `torch.distributed.checkpoint` directory with top-level keys
`model`, `optimizer`, `dataloader`, `lr_scheduler` (+ user states), next to a `config.json` that
rebuilds the model. Saves can be triggered by step interval or by wall-clock interval (agreed
across ranks), run synchronously, through `dcp.async_save`, or staged to pinned host memory on a
side stream and written by a background thread. `keep_latest_k` prunes old steps; `load(-1)`
picks the newest complete step.
"""

from __future__ import annotations

import enum
import os
import re
import shutil
import threading
import time
from typing import Any

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp

from halite_b200.distributed.managers import LRSchedulerManager, ModelManager, OptimizerManager
from halite_b200.logging import logger
from halite_b200.utils import get_torch_dtype


class IntervalType(enum.Enum):
    STEPS = "steps"
    SECONDS = "seconds"


class AsyncMode(str, enum.Enum):
    DISABLED = "disabled"
    ASYNC = "async"
    ASYNC_WITH_PINNED_MEM = "async_with_pinned_mem"


def _state_dict_of(states):
    return {k: (v.state_dict() if hasattr(v, "state_dict") else v) for k, v in states.items()}


class CheckpointManager:
    def __init__(self, model_parts, optimizers, lr_schedulers, dataloader=None, model_config: Any | None = None,
                 states: dict | None = None, directory: str = "checkpoint", interval_type: str = "steps",
                 interval: int = 500, enable_checkpoint: bool = True, keep_latest_k: int = 0,
                 model_weights_only: bool = False, export_dtype: str = "float32", async_mode: str = "disabled"):
        self.enable_checkpoint = enable_checkpoint
        self.keep_latest_k = keep_latest_k
        self.pre_save = None      # optional callable run right before a save that is going to happen
        if not enable_checkpoint:
            return
        self.states = dict(states or {})
        model_mgr = model_parts if isinstance(model_parts, ModelManager) else ModelManager(model_parts)
        optim_mgr = optimizers if isinstance(optimizers, OptimizerManager) else \
            OptimizerManager(model_mgr.models, optimizers)
        self.states.update({"model": model_mgr, "optimizer": optim_mgr})
        if dataloader is not None:
            self.states["dataloader"] = dataloader
        if lr_schedulers is not None:
            sched = lr_schedulers if isinstance(lr_schedulers, LRSchedulerManager) else \
                LRSchedulerManager(optim_mgr, lr_schedulers)
            self.states.update(sched.get_state_dict())
        self.model_config = model_config
        self.directory = directory
        self.interval_type = IntervalType.SECONDS if interval_type == "seconds" else IntervalType.STEPS
        self.interval = interval
        self.begin_time = time.monotonic()
        self.model_weights_only = model_weights_only
        self.export_dtype = get_torch_dtype(export_dtype)
        self.async_mode = AsyncMode(async_mode.lower())
        self._future = None
        self._thread = None
        self._pg = None
        if dist.is_initialized():
            self._pg = dist.new_group(backend="gloo")

    # ------------------------------------------------------------------ helpers
    def reset(self):
        self.begin_time = time.monotonic()

    def _id(self, step):
        return os.path.join(self.directory, f"step-{step}")

    def _rank(self):
        return dist.get_rank() if dist.is_initialized() else 0

    def _should_save(self, step, force=False):
        if not self.enable_checkpoint:
            return False
        if force:
            return True
        if self.interval_type == IntervalType.STEPS:
            return self.interval > 0 and step % self.interval == 0
        # wall-clock interval: every rank must reach the same decision
        elapsed = torch.tensor([time.monotonic() - self.begin_time], dtype=torch.float64)
        if self._pg is not None:
            dist.all_reduce(elapsed, op=dist.ReduceOp.MIN, group=self._pg)
        return float(elapsed) >= self.interval

    def _wait(self):
        if self._future is not None:
            self._future.result()
            self._future = None
        if self._thread is not None:
            self._thread.join()
            self._thread = None

    def _write_config(self, path):
        if self.model_config is None or self._rank() != 0:
            return
        os.makedirs(path, exist_ok=True)
        if hasattr(self.model_config, "save"):
            self.model_config.save(path)

    # ------------------------------------------------------------------ save
    def save(self, step: int, force: bool = False, last: bool = False):
        if not self._should_save(step, force):
            return False
        if self.pre_save is not None:
            self.pre_save()
        self._wait()
        path = self._id(step)
        if last and self.model_weights_only:
            sd = self.states["model"].state_dict()
            if self.export_dtype != torch.float32:
                sd = {k: v.to(self.export_dtype) for k, v in sd.items()}
            dcp.save({"model": sd}, checkpoint_id=path)
        else:
            sd = _state_dict_of(self.states)
            if self.async_mode == AsyncMode.ASYNC:
                self._future = dcp.async_save(sd, checkpoint_id=path, process_group=self._pg)
            elif self.async_mode == AsyncMode.ASYNC_WITH_PINNED_MEM and torch.cuda.is_available():
                staged = self._stage_to_host(sd)
                if staged is None:
                    self._future = dcp.async_save(sd, checkpoint_id=path, process_group=self._pg)
                else:
                    self._thread = threading.Thread(
                        target=dcp.save, args=(staged,),
                        kwargs={"checkpoint_id": path, "process_group": self._pg}, daemon=True)
                    self._thread.start()
            else:
                dcp.save(sd, checkpoint_id=path)
        self._write_config(path)
        self.reset()
        self._purge(step)
        return True

    def _stage_to_host(self, sd):
        """Copy device tensors to pinned host memory on a side stream and return the host copy
        for the writer thread; training continues once the copies have landed. Returns None when
        the state holds sharded (DTensor) entries, which go through `dcp.async_save` instead."""
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        sharded = False

        def move(x):
            nonlocal sharded
            if hasattr(x, "to_local"):
                sharded = True
                return x
            if isinstance(x, torch.Tensor) and x.is_cuda:
                host = torch.empty(x.shape, dtype=x.dtype, pin_memory=True)
                host.copy_(x, non_blocking=True)
                return host
            if isinstance(x, dict):
                return {k: move(v) for k, v in x.items()}
            return x

        with torch.cuda.stream(stream):
            out = move(sd)
        stream.synchronize()
        return None if sharded else out

    def _purge(self, current=None):
        if self.keep_latest_k <= 0 or self._rank() != 0 or not os.path.isdir(self.directory):
            return
        # a save still in flight may not have created its folder yet: count it anyway
        steps = sorted(set(self._steps(complete_only=False)) | ({current} if current is not None else set()))
        for s in steps[: -self.keep_latest_k]:
            shutil.rmtree(self._id(s), ignore_errors=True)

    # ------------------------------------------------------------------ load
    def _steps(self, complete_only=True):
        out = []
        if not os.path.isdir(self.directory):
            return out
        for name in os.listdir(self.directory):
            m = re.fullmatch(r"step-(\d+)", name)
            if m and (not complete_only or os.path.exists(os.path.join(self.directory, name, ".metadata"))):
                out.append(int(m.group(1)))
        return out

    def _adapt_to_saved_sizes(self, sd, path):
        """Flat shards saved under a shard count whose padded length differs from the current one
        cannot be resharded by the planner: read such an entry whole and cut this rank's range
        out of it afterwards (the padding holds no state)."""
        meta = dcp.FileSystemReader(path).read_metadata().state_dict_metadata
        fixups = []
        for group, entries in sd.items():
            if not isinstance(entries, dict):
                continue
            for key, val in list(entries.items()):
                saved = meta.get(f"{group}.{key}")
                if isinstance(val, torch.Tensor) and val.dim() == 1 and saved is not None \
                        and hasattr(saved, "size") and tuple(saved.size) != tuple(val.shape):
                    local = val.to_local() if hasattr(val, "to_local") else val
                    full = torch.empty(tuple(saved.size), dtype=local.dtype, device=local.device)
                    entries[key] = full
                    fixups.append((group, key, val, full))
        return fixups

    def load(self, step: int = -1) -> bool:
        if not self.enable_checkpoint:
            return False
        self._wait()
        if step == -1:
            steps = self._steps()
            if not steps:
                return False
            step = max(steps)
        path = self._id(step)
        if not os.path.exists(os.path.join(path, ".metadata")):
            return False
        # step 0 is a converted / pretrained model: weights only
        keys = ["model"] if step == 0 else list(self.states.keys())
        sd = {k: (self.states[k].state_dict() if hasattr(self.states[k], "state_dict") else self.states[k])
              for k in keys}
        # state that a fresh object has not created yet (lazily built optimizer state) is asked
        # for by the checkpoint's own key list, not by the fresh object's
        saved_meta = dcp.FileSystemReader(path).read_metadata().state_dict_metadata
        for k in keys:
            if hasattr(self.states[k], "extend_load_template") and isinstance(sd[k], dict):
                self.states[k].extend_load_template(
                    sd[k], {key[len(k) + 1:]: md for key, md in saved_meta.items() if key.startswith(k + ".")})
        fixups = self._adapt_to_saved_sizes(sd, path)
        dcp.load(sd, checkpoint_id=path)
        for group, key, original, full in fixups:
            local = original.to_local() if hasattr(original, "to_local") else original
            rank = original.device_mesh.get_local_rank() if hasattr(original, "to_local") else 0
            lo = rank * local.numel()
            n = max(0, min(local.numel(), full.numel() - lo))
            local.zero_()
            local[:n].copy_(full[lo:lo + n])
            sd[group][key] = original
        for k in keys:
            if hasattr(self.states[k], "load_state_dict"):
                self.states[k].load_state_dict(sd[k])
        logger.info(f"loaded checkpoint {path}")
        return True


def load_checkpoint(model, checkpoint_path, strict=True):
    """Load model weights from a DCP directory whose top-level key is `model`."""
    mgr = ModelManager(model)
    sd = {"model": mgr.state_dict()}
    dcp.load(sd, checkpoint_id=checkpoint_path)
    mgr.load_state_dict(sd["model"])
    return model
