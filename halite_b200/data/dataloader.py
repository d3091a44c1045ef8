"""Resumable data loading (reference: data/dataloader.py:15-130, data/simple_dataloader.py:15-232).

`DataLoader` batches a stateful iterable dataset, optionally through worker processes. Every
sample leaves its worker together with a snapshot of that worker's dataset state; the loader's
`state_dict()` is the set of snapshots behind the last batch it returned, so a resumed loader
replays nothing and skips nothing. `DataManager` makes all data-parallel ranks stop at the same
step (a MAX all-reduce of a "finished" flag per step).
"""

from __future__ import annotations

import copy
import multiprocessing as mp
import pickle
import queue as queue_mod
import random

import torch
import torch.distributed as dist
from torch.utils.data._utils.worker import WorkerInfo


def _worker_loop(q, stop, dataset, worker_id, n_workers, seed, state):
    torch.utils.data._utils.worker._worker_info = WorkerInfo(
        id=worker_id, num_workers=n_workers, seed=seed + worker_id, dataset=dataset)
    random.seed(seed + worker_id)
    torch.manual_seed(seed + worker_id)
    torch.set_num_threads(1)
    if state is not None and hasattr(dataset, "load_state_dict"):
        dataset.load_state_dict(state)
    has_state = hasattr(dataset, "state_dict")
    for item in dataset:
        snap = copy.deepcopy(dataset.state_dict()) if has_state else None
        while not stop.is_set():
            try:
                q.put((item, False, snap), timeout=0.1)
                break
            except queue_mod.Full:
                continue
        if stop.is_set():
            break
    try:
        q.put((None, True, None), timeout=1.0)
    except queue_mod.Full:
        pass
    stop.wait()


class DataLoader:
    def __init__(self, dataset, batch_size=1, rank=0, num_workers=0, collate_fn=None, drop_last=True,
                 prefetch_factor=2, seed=0, pin_memory=False, **unused):
        self.dataset = dataset
        self.batch_size = batch_size
        self.rank = rank
        self.num_workers = num_workers
        self.collate_fn = collate_fn or torch.utils.data.default_collate
        self.drop_last = drop_last
        self.prefetch = max(1, prefetch_factor) * max(1, batch_size)
        self.seed = seed
        self.pin_memory = pin_memory
        self._rank_id = f"dp_rank_{rank}"
        self._worker_states = {}       # worker id -> dataset state behind the last returned batch
        self._next_worker = 0
        self._finished = set()
        self._resume = None
        self._procs, self._queues, self._stop = [], [], None

    def __len__(self):
        return len(self.dataset) // max(1, getattr(self.dataset, "num_replicas", 1)) // self.batch_size

    # ------------------------------------------------------------------ state
    def state_dict(self):
        if self.num_workers == 0:
            inner = self.dataset.state_dict() if hasattr(self.dataset, "state_dict") else None
            state = {"dataset": copy.deepcopy(inner)}
        else:
            state = {"workers": copy.deepcopy(self._worker_states), "next_worker": self._next_worker,
                     "finished": sorted(self._finished)}
        return {self._rank_id: pickle.dumps(state)}

    def load_state_dict(self, state_dict):
        if not state_dict or self._rank_id not in state_dict:
            return
        self._resume = pickle.loads(state_dict[self._rank_id])
        if self.num_workers == 0 and self._resume.get("dataset") is not None:
            self.dataset.load_state_dict(self._resume["dataset"])

    # ------------------------------------------------------------------ iteration
    def _finish(self, batch):
        out = self.collate_fn(batch)
        if self.pin_memory and hasattr(out, "pin_memory"):
            out = out.pin_memory()
        return out

    def __iter__(self):
        if self.num_workers == 0:
            yield from self._iter_inline()
        else:
            yield from self._iter_workers()

    def _iter_inline(self):
        batch = []
        for item in self.dataset:
            batch.append(item)
            if len(batch) == self.batch_size:
                yield self._finish(batch)
                batch = []
        if batch and not self.drop_last:
            yield self._finish(batch)

    def _start_workers(self):
        ctx = mp.get_context("fork")
        self._stop = ctx.Event()
        resume = self._resume or {}
        states = resume.get("workers", {})
        self._next_worker = resume.get("next_worker", 0)
        self._finished = set(resume.get("finished", []))
        self._worker_states = dict(states)
        self._queues, self._procs = [], []
        for w in range(self.num_workers):
            q = ctx.Queue(maxsize=self.prefetch)
            p = ctx.Process(target=_worker_loop, daemon=True,
                            args=(q, self._stop, self.dataset, w, self.num_workers, self.seed, states.get(w)))
            p.start()
            self._queues.append(q)
            self._procs.append(p)
        self._resume = None

    def _shutdown(self):
        if self._stop is not None:
            self._stop.set()
        for p in self._procs:
            p.join(timeout=2)
            if p.is_alive():
                p.terminate()
        self._procs, self._queues, self._stop = [], [], None

    def _iter_workers(self):
        self._start_workers()
        try:
            batch, pending = [], {}
            while len(self._finished) < self.num_workers:
                w = self._next_worker
                self._next_worker = (w + 1) % self.num_workers
                if w in self._finished:
                    continue
                while True:
                    try:
                        item, done, snap = self._queues[w].get(timeout=0.1)
                        break
                    except queue_mod.Empty:
                        if not self._procs[w].is_alive() and self._queues[w].empty():
                            raise RuntimeError(f"data worker {w} died")
                if done:
                    self._finished.add(w)
                    continue
                batch.append(item)
                pending[w] = snap
                if len(batch) == self.batch_size:
                    self._worker_states.update(pending)
                    pending = {}
                    yield self._finish(batch)
                    batch = []
            if batch and not self.drop_last:
                self._worker_states.update(pending)
                yield self._finish(batch)
        finally:
            self._shutdown()


SimpleDataLoader = DataLoader


class DataManager:
    """Iterates one or several loaders in sequence; with `check_finished` every rank of
    `process_group` stops at the step where the first rank runs out."""

    def __init__(self, loaders, process_group=None, check_finished=True, device=None):
        self.loaders = list(loaders) if isinstance(loaders, (list, tuple)) else [loaders]
        self.pg = process_group
        self.check_finished = check_finished and dist.is_initialized()
        if device is None:
            device = "cuda" if torch.cuda.is_available() and dist.is_initialized() and \
                dist.get_backend(process_group) != "gloo" else "cpu"
        self.flag = torch.zeros(1, dtype=torch.float32, device=device)

    def __iter__(self):
        self._iters = iter(self.loaders)
        self._cur = iter(next(self._iters))
        return self

    def __next__(self):
        batch, finished = None, False
        while True:
            try:
                batch = next(self._cur)
                break
            except StopIteration:
                nxt = next(self._iters, None)
                if nxt is None:
                    finished = True
                    break
                self._cur = iter(nxt)
        if self.check_finished:
            self.flag.fill_(float(finished))
            dist.all_reduce(self.flag, op=dist.ReduceOp.MAX, group=self.pg)
            finished = bool(self.flag.item() > 0)
        if finished:
            raise StopIteration
        return batch
