"""Asynchronous, disaggregated rollout generation (reference: projects/common/rollout_monarch.py
and scripts/ppo_monarch.py, which build on the Monarch actor library).

Here the actors are plain processes of one job. Ranks [0, T) train; ranks [T, T+G) generate. All
of them join one `StatelessProcessGroup` (a TCP store) for control messages, rollouts and, on
CPU, weights; on GPUs weights travel by an NCCL broadcast over a communicator created next to
`torch.distributed`'s own groups. Generators run their engine continuously: between engine
calls they poll for a newer policy, so weights change mid-run; every rollout is stamped with the
policy version that produced it and the replay buffer drops rollouts that are too stale.
"""

from __future__ import annotations

import math
import threading
import time
from collections import deque
from typing import NamedTuple

import torch


class FinishedGeneration:
    pass


class Empty:
    pass


class TensorSpec(NamedTuple):
    """What a receiver must allocate for one tensor of a weight transfer."""

    name: str
    shape: tuple
    dtype: torch.dtype

    @staticmethod
    def from_tensor(name, tensor):
        return TensorSpec(name, tuple(tensor.shape), tensor.dtype)

    def empty(self, device):
        return torch.empty(self.shape, dtype=self.dtype, device=device)


def get_peer_ranks(rank, size, target_size, overlap_targets=False):
    """Which ranks of a `target_size` group rank `rank` of a `size` group talks to."""
    if size == target_size:
        return [rank]
    if size < target_size:
        step = math.ceil(target_size / size)
        return [r for r in range(rank * step, (rank + 1) * step) if r < target_size]
    if not overlap_targets:
        return [rank] if rank < target_size else []
    return [rank % target_size]


def chunk_list(xs, n_chunk):
    """Split into `n_chunk` nearly equal consecutive parts (the first parts get the remainder)."""
    size, rem = divmod(len(xs), n_chunk)
    out, start = [], 0
    for i in range(n_chunk):
        end = start + size + (1 if i < rem else 0)
        out.append(xs[start:end])
        start = end
    return out


def infinite_loader(loader):
    while True:
        yield from loader


class ReplayBuffer:
    """Thread-safe FIFO of (policy_version, rollouts) groups with a staleness bound."""

    def __init__(self, capacity: int = 64, max_staleness: int = 1):
        self.capacity, self.max_staleness = capacity, max_staleness
        self._items: deque = deque()
        self._cond = threading.Condition()
        self.dropped = 0

    def put(self, version, rollouts):
        with self._cond:
            self._items.append((version, rollouts))
            while len(self._items) > self.capacity:
                self._items.popleft()
                self.dropped += 1
            self._cond.notify_all()

    def get(self, current_version, timeout=None):
        """Oldest group that is at most `max_staleness` versions old; older ones are discarded."""
        deadline = None if timeout is None else time.monotonic() + timeout
        with self._cond:
            while True:
                while self._items and current_version - self._items[0][0] > self.max_staleness:
                    self._items.popleft()
                    self.dropped += 1
                if self._items:
                    return self._items.popleft()
                remaining = None if deadline is None else deadline - time.monotonic()
                if remaining is not None and remaining <= 0:
                    raise TimeoutError("no rollouts arrived")
                self._cond.wait(remaining)

    def __len__(self):
        with self._cond:
            return len(self._items)


class BidirectionalQueue:
    """Message pair between two ranks over the stateless group."""

    def __init__(self, group, peer):
        self.group, self.peer = group, peer

    def put(self, obj):
        self.group.send_obj(obj, self.peer)

    def get(self):
        return self.group.recv_obj(self.peer)


class WeightChannel:
    """Policy weights from trainer rank 0 to every generator. `comm`: a `PyNcclCommunicator` over
    {trainer 0} + generators for device tensors, or None to ship CPU tensors through the store."""

    def __init__(self, group, trainer_rank, generator_ranks, comm=None):
        self.group, self.trainer_rank, self.generator_ranks, self.comm = group, trainer_rank, list(generator_ranks), comm

    def push(self, state_dict, version):
        specs = [TensorSpec.from_tensor(k, v) for k, v in state_dict.items()]
        if self.comm is None:
            payload = {k: v.detach().to("cpu") for k, v in state_dict.items()}
            for g in self.generator_ranks:
                self.group.send_obj(("weights", version, specs, payload), g)
            return
        for g in self.generator_ranks:
            self.group.send_obj(("weights", version, specs, None), g)
        for k, v in state_dict.items():
            self.comm.broadcast(v.detach().contiguous(), src=0)

    def receive(self, message, device):
        _, version, specs, payload = message
        if payload is not None:
            return version, {k: v.to(device) for k, v in payload.items()}
        out = {}
        for spec in specs:
            t = spec.empty(device)
            self.comm.broadcast(t, src=0)
            out[spec.name] = t
        return version, out


class EnvironmentWorker:
    """Scores finished generations (the reward registry lives inside the rollout generator)."""

    def __init__(self, rollout_generator):
        self.rollout_generator = rollout_generator

    def score(self, rollouts, output_ids, output_logprobs=None):
        return self.rollout_generator.build_rollout(rollouts, output_ids, output_logprobs)


class GeneratorWorker:
    """Loop of a generator rank: take a prompt batch, generate, score, send the rollouts back to
    trainer 0; between batches (and between engine calls within a batch when the batch is split)
    adopt newer weights."""

    def __init__(self, group, rank, trainer_rank, engine, rollout_generator, request_builder, weights: WeightChannel,
                 device="cpu", generation_chunk=None):
        self.group, self.rank, self.trainer_rank = group, rank, trainer_rank
        self.engine, self.rollout_generator, self.request_builder = engine, rollout_generator, request_builder
        self.env = EnvironmentWorker(rollout_generator)
        self.weights, self.device = weights, device
        self.version = -1
        self.generation_chunk = generation_chunk
        self.batches_done = 0

    def _adopt(self, message):
        self.version, sd = self.weights.receive(message, self.device)
        self.engine.load_state_dict(sd)

    def run(self):
        pending = deque()
        while True:
            msg = self.group.recv_obj(self.trainer_rank) if not pending else pending.popleft()
            kind = msg[0]
            if kind == "stop":
                break
            if kind == "weights":
                self._adopt(msg)
                continue
            if kind != "prompts":
                raise ValueError(f"unexpected message {kind}")
            batch = msg[1]
            rollouts = self.request_builder(batch)
            chunks = [rollouts] if not self.generation_chunk else \
                [rollouts[i:i + self.generation_chunk] for i in range(0, len(rollouts), self.generation_chunk)]
            done = []
            for chunk in chunks:
                results = self.engine.infer_batch([r.to_inference_request() for r in chunk])
                by_id = {res.id: res for res in results}
                ids = [by_id[r.id].output_ids for r in chunk]
                lps = [by_id[r.id].output_logprobs for r in chunk]
                scored = self.env.score(chunk, ids, lps if all(l for l in lps) else None)
                done.extend(scored)
            for r in done:
                r.state["policy_version"] = self.version
            self.group.send_obj(("rollouts", self.rank, self.version, done), self.trainer_rank)
            self.batches_done += 1


class RolloutManager:
    """Runs on trainer rank 0: keeps every generator supplied with prompt batches and moves the
    returned rollouts into the replay buffer. One feeder thread per generator."""

    def __init__(self, group, generator_ranks, prompt_iter, buffer: ReplayBuffer):
        self.group, self.generator_ranks = group, list(generator_ranks)
        self.prompts, self.buffer = prompt_iter, buffer
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self.threads = []
        self.pushed_versions = {g: -1 for g in self.generator_ranks}
        self._outbox = {g: deque() for g in self.generator_ranks}

    def _next_prompts(self):
        with self._lock:
            return next(self.prompts, None)

    def queue_weights(self, message_builder):
        """Ask every feeder to forward a weight update before its next prompt batch."""
        for g in self.generator_ranks:
            self._outbox[g].append(message_builder)

    def _feed(self, g):
        while not self._stop.is_set():
            while self._outbox[g]:
                self._outbox[g].popleft()(g)
            batch = self._next_prompts()
            if batch is None:
                break
            self.group.send_obj(("prompts", batch), g)
            tag, rank, version, rollouts = self.group.recv_obj(g)
            assert tag == "rollouts" and rank == g
            self.buffer.put(version, rollouts)
        self.group.send_obj(("stop",), g)

    def start(self):
        for g in self.generator_ranks:
            t = threading.Thread(target=self._feed, args=(g,), daemon=True)
            t.start()
            self.threads.append(t)

    def stop(self):
        self._stop.set()
        for t in self.threads:
            t.join(timeout=60)
