"""Parallel layout of a job: data-parallel replicate / shard, tensor and pipeline degrees
(reference: parallel/parallel_dims.py:7-110). One process per GPU; `torch.distributed`
provides the plumbing (NCCL for CUDA tensors, Gloo for CPU tensors).

Rank order is [pp, dp_replicate, dp_shard, tp] with tp fastest, so TP peers are neighbouring
ranks and FSDP shards stride by tp.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from datetime import timedelta

import torch
import torch.distributed as dist


@dataclass
class ParallelDims:
    dp_replicate: int = 1
    dp_shard: int = -1
    tp: int = 1
    pp: int = 1
    world_size: int | None = None

    def __post_init__(self):
        if self.world_size is None:
            self.world_size = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.rank = int(os.environ.get("RANK", "0"))
        for name in ("dp_replicate", "tp", "pp"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be >= 1")
        if self.dp_shard == -1:
            denom = self.dp_replicate * self.tp * self.pp
            if self.world_size % denom:
                raise ValueError(f"world size {self.world_size} is not divisible by "
                                 f"dp_replicate*tp*pp = {denom}")
            self.dp_shard = self.world_size // denom
        if self.dp_replicate * self.dp_shard * self.tp * self.pp != self.world_size:
            raise ValueError(
                f"dp_replicate({self.dp_replicate}) * dp_shard({self.dp_shard}) * tp({self.tp}) * "
                f"pp({self.pp}) != world size ({self.world_size})")
        self._groups = {}
        self.mesh = None

    # ------------------------------------------------------------------ properties
    @property
    def dp(self):
        return self.dp_replicate * self.dp_shard

    @property
    def dp_enabled(self):
        return self.dp > 1

    @property
    def dp_replicate_enabled(self):
        return self.dp_replicate > 1

    @property
    def dp_shard_enabled(self):
        return self.dp_shard > 1

    @property
    def tp_enabled(self):
        return self.tp > 1

    @property
    def pp_enabled(self):
        return self.pp > 1

    @property
    def is_primary(self):
        return self.rank == 0

    def coords(self, rank=None):
        """(pp, dp_replicate, dp_shard, tp) coordinates of a rank."""
        r = self.rank if rank is None else rank
        tp = r % self.tp
        r //= self.tp
        ds = r % self.dp_shard
        r //= self.dp_shard
        dr = r % self.dp_replicate
        r //= self.dp_replicate
        return r, dr, ds, tp

    @property
    def dp_rank(self):
        _, dr, ds, _ = self.coords()
        return dr * self.dp_shard + ds

    @property
    def tp_rank(self):
        return self.coords()[3]

    # ------------------------------------------------------------------ init
    def initialize(self, timeout_s: float = 600.0):
        """Start the default process group (NCCL + Gloo on a GPU box, Gloo alone on CPU)."""
        if dist.is_initialized():
            return self
        if torch.cuda.is_available():
            torch.cuda.set_device(self.local_rank)
            backend = "cpu:gloo,cuda:nccl"
        else:
            backend = "gloo"
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group(backend, rank=self.rank, world_size=self.world_size,
                                timeout=timedelta(seconds=timeout_s))
        return self

    def build_mesh(self, device_type: str | None = None):
        """Create the process groups of every dimension. Returns self (the object doubles as
        the mesh: `mesh.group("dp_shard")`, `mesh.size("tp")`)."""
        if device_type is None:
            device_type = "cuda" if torch.cuda.is_available() else "cpu"
        self.device_type = device_type
        if self.world_size > 1 and not dist.is_initialized():
            self.initialize()
        self.mesh = self
        if self.world_size == 1:
            return self
        ranks = torch.arange(self.world_size).view(self.pp, self.dp_replicate, self.dp_shard, self.tp)
        names = ("pp", "dp_replicate", "dp_shard", "tp")
        for d, name in enumerate(names):
            moved = ranks.movedim(d, -1).reshape(-1, ranks.shape[d])
            for row in moved.tolist():
                g = dist.new_group(row) if len(row) > 1 else None
                if self.rank in row:
                    self._groups[name] = (g, row)
        # flattened data-parallel group (replicate x shard)
        dp = ranks.permute(0, 3, 1, 2).reshape(-1, self.dp_replicate * self.dp_shard)
        for row in dp.tolist():
            g = dist.new_group(row) if len(row) > 1 else None
            if self.rank in row:
                self._groups["dp"] = (g, row)
        return self

    def group(self, name):
        """Process group of a mesh dimension, None when that dimension has size 1."""
        if name not in self._groups:
            return None
        return self._groups[name][0]

    def group_ranks(self, name):
        if name not in self._groups:
            return [self.rank]
        return self._groups[name][1]

    def size(self, name):
        return {"pp": self.pp, "dp_replicate": self.dp_replicate, "dp_shard": self.dp_shard,
                "tp": self.tp, "dp": self.dp}[name]

    def local_rank_in(self, name):
        return self.group_ranks(name).index(self.rank)
