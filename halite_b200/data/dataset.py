"""Datasets (reference: data/dataset.py:152-371): shard specs -> sources, map-style and
weighted iterable datasets with deterministic shuffling, rank / worker striding and exact
resume, plus the synthetic token stream used by benchmarks."""

from __future__ import annotations

import bisect
import math
import os

import torch
from torch.utils import data

from halite_b200.data.index_shuffle import index_shuffle
from halite_b200.data.record import Record
from halite_b200.data.sources import FileInstruction, open_source


def build_dataset_from_spec(spec, split="train", split_ratio=0):
    """spec: {root, ratios: {name: w}, shards: {name: {file: n_records}}}.

    `train` reads the last `split_ratio` share of every shard (at least one record; the whole
    shard when the ratio is 0), any other split reads the first `split_ratio` share (rounded up).
    With train_ratio + eval_ratio <= 1 the two never overlap."""
    get = spec.get if hasattr(spec, "get") else lambda k: getattr(spec, k)
    sources, ratios, names = [], [], []
    for name, shards in get("shards").items():
        instructions = []
        for shard, size in shards.items():
            path = os.path.join(get("root"), name, shard)
            if split == "train":
                take = max(math.floor(size * split_ratio), 1) if split_ratio else size
                instructions.append(FileInstruction(path, size - take, take, size))
            else:
                take = max(math.ceil(size * split_ratio), 1) if split_ratio else 0
                instructions.append(FileInstruction(path, 0, take, size))
        if not instructions:
            continue
        sources.append(open_source(instructions))
        ratios.append(get("ratios")[name])
        names.append(name)
    return sources, ratios, names


def _record(source, dataset_idx, sample_idx, names):
    return Record(data=source[sample_idx % len(source)],
                  _meta_={"dataset_id": dataset_idx, "sample_id": sample_idx,
                          "dataset_name": names[dataset_idx] if names is not None else None})


class MapDataset(data.Dataset):
    def __init__(self, datasets, names=None, operations=None):
        self.datasets = datasets
        self.names = names
        self.points = torch.cumsum(torch.tensor([len(d) for d in datasets]), 0).tolist()
        self.operations = operations or []

    def __len__(self):
        return self.points[-1]

    def __getitem__(self, idx):
        d = bisect.bisect_right(self.points, idx)
        local = idx - (self.points[d - 1] if d else 0)
        stream = [_record(self.datasets[d], d, local, self.names)]
        for op in self.operations:
            stream = op(stream)
        return next(iter(stream))


def HFDataset(path, name=None, split="test", operations=None):
    from datasets import load_dataset

    return MapDataset([load_dataset(path, name, split=split)], operations=operations)


class WeightedIterableDataset(data.IterableDataset):
    """Mixes sources by ratio: source i contributes `target_sample[i]` indices per epoch (wrapping
    around when upsampled). Position p of the epoch maps through `index_shuffle` to a (source,
    sample) pair, ranks take contiguous blocks and workers stride inside them, so
    `state_dict()` (= next position + per-op states) resumes the exact stream."""

    def __init__(self, datasets, ratios, names=None, operations=None, num_replicas=1, rank=0,
                 upsample=False, shuffle=True, seed=42, ensure_divisible_to=1):
        self.datasets = datasets
        self.names = names
        self.ratios = list(ratios)
        self.num_replicas, self.rank = num_replicas, rank
        sizes = torch.tensor([len(d) for d in datasets], dtype=torch.float64)
        r = torch.tensor(self.ratios, dtype=torch.float64)
        want = sizes.sum() * r / r.sum()
        scale = torch.min(want / sizes) if upsample else torch.max(want / sizes)
        target = torch.round(want / scale).to(torch.int64)
        if ensure_divisible_to > 1:
            target = target // ensure_divisible_to * ensure_divisible_to
        self.target_sample = target
        self.points = torch.cumsum(target, 0).tolist()
        self.operations = operations or []
        self.shuffle, self.seed = shuffle, seed
        self._current_id = None
        self._sample_states = {}
        self.worker_state = None

    def __len__(self):
        return self.points[-1]

    def summary(self, total=True):
        rows = []
        for i, (d, ratio, n) in enumerate(zip(self.datasets, self.ratios, self.target_sample.tolist())):
            name = f" {self.names[i]}" if self.names is not None else ""
            rows.append(f"#{i}{name} size: {len(d)} ratio: {ratio} sample: {n}")
        if total:
            rows.append(f"total: {len(self)}")
        return "\n".join(rows)

    def __getitem__(self, idx):
        if self.shuffle:
            idx = index_shuffle(idx, len(self) - 1, self.seed, 4)
        d = bisect.bisect_right(self.points, idx)
        local = idx - (self.points[d - 1] if d else 0)
        return _record(self.datasets[d], d, local, self.names)

    def set_worker_state(self, worker_info):
        offset, step = (0, 1) if worker_info is None else (worker_info.id, worker_info.num_workers)
        per_rank = len(self) // self.num_replicas
        start = per_rank * self.rank + offset
        self.worker_state = {"start": start, "end": per_rank * (self.rank + 1), "step": step,
                             "worker_id": offset, "num_workers": step, "dp_rank": self.rank,
                             "dp_size": self.num_replicas, "seed": self.seed}
        if self._current_id is None:
            self._current_id = start

    def state_dict(self):
        return {"current_id": self._current_id, "sample_states": dict(self._sample_states)}

    def load_state_dict(self, state):
        self._current_id = state["current_id"]
        self._sample_states = dict(state["sample_states"])
        for i, op in enumerate(self.operations):
            if i in self._sample_states and hasattr(op, "load_state_dict"):
                op.load_state_dict(self._sample_states[i])

    def sample_iterator(self):
        ws = self.worker_state
        for idx in range(self._current_id, ws["end"], ws["step"]):
            rec = self[idx]
            self._current_id = idx + ws["step"]
            yield rec

    def __iter__(self):
        self.set_worker_state(data.get_worker_info())
        stream = self.sample_iterator()
        for op in self.operations:
            stream = op(stream)
        for sample in stream:
            for i, op in enumerate(self.operations):
                if hasattr(op, "state_dict"):
                    self._sample_states[i] = op.state_dict()
            yield sample


class SyntheticTokenDataset(data.IterableDataset):
    """Endless stream of uniform-random token sequences, seeded per (rank, position): the data of
    the benchmark configs. Yields {"input": [S], "target": [S]}."""

    def __init__(self, vocab_size, seq_len, seed=0, rank=0, num_replicas=1, length=None):
        self.vocab_size, self.seq_len = vocab_size, seq_len
        self.seed, self.rank, self.num_replicas = seed, rank, num_replicas
        self.length = length
        self._pos = 0

    def state_dict(self):
        return {"pos": self._pos}

    def load_state_dict(self, state):
        self._pos = state["pos"]

    def __iter__(self):
        while self.length is None or self._pos < self.length:
            g = torch.Generator().manual_seed(self.seed * 1000003 + self.rank * 7919 + self._pos)
            t = torch.randint(0, self.vocab_size, (self.seq_len + 1,), generator=g)
            self._pos += 1
            yield Record(input=t[:-1], target=t[1:])
