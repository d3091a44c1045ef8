"""Process groups that leave `torch.distributed`'s global state alone
(reference: distributed/process_group.py:52-672).

`StatelessProcessGroup` is a metadata plane over a `TCPStore`: object send / recv / broadcast /
all-gather and a barrier that raises instead of hanging. `PyNcclCommunicator` builds an NCCL
communicator of its own from a unique id passed over that plane, with the collectives a weight
transfer needs (including the uneven all-gatherv / reduce-scatterv as grouped broadcasts /
reduces).
"""

from __future__ import annotations

import pickle
import threading
import time
from collections import deque
from datetime import timedelta
from typing import Any

import torch
from torch.distributed import ReduceOp, TCPStore

from halite_b200.distributed.pynccl_wrapper import (NCCLLibrary, buffer_t, cudaStream_t, ncclDataTypeEnum,
                                                    ncclRedOpTypeEnum)


class StatelessProcessGroup:
    def __init__(self, rank: int, world_size: int, store, data_expiration_seconds: int = 3600):
        if not 0 <= rank < world_size:
            raise ValueError("rank out of range")
        self.rank, self.world_size, self.store = rank, world_size, store
        self.data_expiration_seconds = data_expiration_seconds
        self._send = [0] * world_size
        self._recv = [0] * world_size
        self._bcast_sent = 0
        self._bcast_recv = [0] * world_size
        self._barriers = 0
        self._entries: deque = deque()
        self._lock = threading.Lock()      # several threads may send (each to its own peer)

    @classmethod
    def create(cls, host: str, port: int, rank: int, world_size: int, data_expiration_seconds: int = 3600,
               store_timeout: float = 300.0):
        store = TCPStore(host_name=host, port=port, world_size=world_size, is_master=rank == 0,
                         timeout=timedelta(seconds=store_timeout))
        return cls(rank, world_size, store, data_expiration_seconds)

    # ------------------------------------------------------------------ bookkeeping
    def _put(self, key, obj):
        data = pickle.dumps(obj)
        with self._lock:
            self.expire_data()
            self.store.set(key, data)
            self._entries.append((key, time.time()))

    def expire_data(self):
        now = time.time()
        while self._entries and now - self._entries[0][1] > self.data_expiration_seconds:
            self.store.delete_key(self._entries.popleft()[0])

    # ------------------------------------------------------------------ objects
    def send_obj(self, obj: Any, dst: int):
        self._put(f"p2p/{self.rank}->{dst}/{self._send[dst]}", obj)
        self._send[dst] += 1

    def recv_obj(self, src: int) -> Any:
        obj = pickle.loads(self.store.get(f"p2p/{src}->{self.rank}/{self._recv[src]}"))
        self._recv[src] += 1
        return obj

    def broadcast_obj(self, obj: Any, src: int) -> Any:
        if self.rank == src:
            self._put(f"bcast/{src}/{self._bcast_sent}", obj)
            self._bcast_sent += 1
            return obj
        out = pickle.loads(self.store.get(f"bcast/{src}/{self._bcast_recv[src]}"))
        self._bcast_recv[src] += 1
        return out

    def all_gather_obj(self, obj: Any) -> list:
        return [self.broadcast_obj(obj if r == self.rank else None, src=r) for r in range(self.world_size)]

    # ------------------------------------------------------------------ barrier
    def barrier(self, timeout: float = 30.0):
        """Arrive, wait until everyone has arrived, then wait until everyone has seen that
        (so the keys can be deleted safely). Raises RuntimeError when `timeout` seconds pass."""
        bid = self._barriers
        self._barriers += 1
        deadline = time.time() + timeout

        def wait_count(prefix):
            self.store.set(f"{prefix}/{self.rank}", b"1")
            keys = [f"{prefix}/{r}" for r in range(self.world_size)]
            pending = list(keys)
            while pending:
                pending = [k for k in pending if not self.store.check([k])]
                if pending:
                    if time.time() > deadline:
                        raise RuntimeError(f"barrier {bid} timed out after {timeout} s; missing ranks: "
                                           f"{[k.rsplit('/', 1)[1] for k in pending]}")
                    time.sleep(0.01)
            return keys

        arrive = wait_count(f"barrier/{bid}/arrive")
        depart = wait_count(f"barrier/{bid}/depart")
        if self.rank == 0:
            # a last phase so rank 0 deletes only after every rank has passed `depart`
            done = [f"barrier/{bid}/done/{r}" for r in range(1, self.world_size)]
            pending = list(done)
            while pending and time.time() <= deadline:
                pending = [k for k in pending if not self.store.check([k])]
                time.sleep(0.005)
            for k in arrive + depart + done:
                try:
                    self.store.delete_key(k)
                except Exception:  # noqa: BLE001
                    pass
        else:
            self.store.set(f"barrier/{bid}/done/{self.rank}", b"1")


class PyNcclCommunicator:
    def __init__(self, group: StatelessProcessGroup, device, library_path: str | None = None):
        self.group = group
        self.rank, self.world_size = group.rank, group.world_size
        self.device = torch.device(device) if not isinstance(device, int) else torch.device("cuda", device)
        self.available = self.world_size > 1
        self.disabled = not self.available
        if not self.available:
            return
        self.nccl = NCCLLibrary(library_path)
        uid = self.nccl.ncclGetUniqueId() if self.rank == 0 else None
        payload = group.broadcast_obj(bytes(uid.internal) if uid is not None else None, src=0)
        self.unique_id = self.nccl.unique_id_from_bytes(payload)
        with torch.cuda.device(self.device):
            self.comm = self.nccl.ncclCommInitRank(self.world_size, self.unique_id, self.rank)
            warm = torch.zeros(1, device=self.device)
            self.all_reduce(warm)
            torch.cuda.current_stream().synchronize()

    # ------------------------------------------------------------------ helpers
    def _stream(self, stream):
        stream = stream or torch.cuda.current_stream(self.device)
        return cudaStream_t(stream.cuda_stream)

    def _check(self, *tensors):
        for t in tensors:
            if t.device != self.device:
                raise ValueError(f"communicator is bound to {self.device}, got a tensor on {t.device}")

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, tensor, op=ReduceOp.SUM, stream=None, out=None):
        if self.disabled:
            return tensor
        out = torch.empty_like(tensor) if out is None else out
        self._check(tensor, out)
        self.nccl.ncclAllReduce(buffer_t(tensor.data_ptr()), buffer_t(out.data_ptr()), tensor.numel(),
                                ncclDataTypeEnum.from_torch(tensor.dtype), ncclRedOpTypeEnum.from_torch(op),
                                self.comm, self._stream(stream))
        return out

    def all_gather(self, output, input, stream=None):
        if self.disabled:
            return
        self._check(output, input)
        self.nccl.ncclAllGather(buffer_t(input.data_ptr()), buffer_t(output.data_ptr()), input.numel(),
                                ncclDataTypeEnum.from_torch(input.dtype), self.comm, self._stream(stream))

    def all_gatherv(self, output, input, sizes: list[int], stream=None):
        """Ranks contribute `sizes[r]` leading rows each: one grouped set of broadcasts."""
        if self.disabled:
            return
        self._check(output, input)
        s = self._stream(stream)
        row = output[0].numel() if output.dim() > 1 else 1
        self.nccl.ncclGroupStart()
        off = 0
        for root, n in enumerate(sizes):
            dst = output[off:off + n]
            self.nccl.ncclBroadcast(buffer_t(input.data_ptr()), buffer_t(dst.data_ptr()), n * row,
                                    ncclDataTypeEnum.from_torch(input.dtype), root, self.comm, s)
            off += n
        self.nccl.ncclGroupEnd()

    def reduce_scatter(self, output, input, op=ReduceOp.SUM, stream=None):
        if self.disabled:
            return
        self._check(output, input)
        self.nccl.ncclReduceScatter(buffer_t(input.data_ptr()), buffer_t(output.data_ptr()), output.numel(),
                                    ncclDataTypeEnum.from_torch(input.dtype), ncclRedOpTypeEnum.from_torch(op),
                                    self.comm, self._stream(stream))

    def reduce_scatterv(self, output, input, sizes: list[int], op=ReduceOp.SUM, stream=None):
        if self.disabled:
            return
        self._check(output, input)
        s = self._stream(stream)
        row = input[0].numel() if input.dim() > 1 else 1
        self.nccl.ncclGroupStart()
        off = 0
        for root, n in enumerate(sizes):
            chunk = input[off:off + n]
            self.nccl.ncclReduce(buffer_t(chunk.data_ptr()), buffer_t(output.data_ptr()), n * row,
                                 ncclDataTypeEnum.from_torch(input.dtype), ncclRedOpTypeEnum.from_torch(op), root,
                                 self.comm, s)
            off += n
        self.nccl.ncclGroupEnd()

    def send(self, tensor, dst: int, stream=None):
        if self.disabled:
            return
        self._check(tensor)
        self.nccl.ncclSend(buffer_t(tensor.data_ptr()), tensor.numel(), ncclDataTypeEnum.from_torch(tensor.dtype),
                           dst, self.comm, self._stream(stream))

    def recv(self, tensor, src: int, stream=None):
        if self.disabled:
            return
        self._check(tensor)
        self.nccl.ncclRecv(buffer_t(tensor.data_ptr()), tensor.numel(), ncclDataTypeEnum.from_torch(tensor.dtype),
                           src, self.comm, self._stream(stream))

    def broadcast(self, tensor, src: int, stream=None):
        if self.disabled:
            return
        self._check(tensor)
        self.nccl.ncclBroadcast(buffer_t(tensor.data_ptr()), buffer_t(tensor.data_ptr()), tensor.numel(),
                                ncclDataTypeEnum.from_torch(tensor.dtype), src, self.comm, self._stream(stream))

    def group_start(self):
        self.nccl.ncclGroupStart()

    def group_end(self):
        self.nccl.ncclGroupEnd()

    def destroy(self):
        if not self.disabled and getattr(self, "comm", None) is not None:
            self.nccl.ncclCommDestroy(self.comm)
            self.comm = None


def stateless_init_process_group(master_address, master_port, rank, world_size, device):
    """Metadata plane + NCCL communicator in one call."""
    group = StatelessProcessGroup.create(master_address, master_port, rank, world_size)
    return PyNcclCommunicator(group, device)
