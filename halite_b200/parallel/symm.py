"""Symmetric memory: one buffer per rank that every rank of a group can address directly over
NVLink, plus the flag words the fused compute + collective kernels signal through.

Allocation and handle exchange use `torch.distributed._symmetric_memory` (CUDA virtual memory
handles passed between the local processes; also yields an NVLS multicast address when the
switch supports it). Where that is unavailable the buffer is an ordinary CUDA allocation shared
through CUDA IPC handles gathered over the process group. Everything after set-up is this
package's own kernels reading and writing peer pointers.

Layout of a `SymmetricHeap`: `[ flags (int32 x FLAG_WORDS) | data ... ]`. Flag words are only
ever compared with `>= epoch`, and epochs only grow, so they never need resetting.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

FLAG_WORDS = 4096          # int32 words reserved at the head of every heap
_FLAG_BYTES = FLAG_WORDS * 4


def _enable_peer_access(device, world):
    """Touch every peer once so the runtime enables P2P mappings between the devices."""
    for d in range(torch.cuda.device_count()):
        if d != device.index:
            try:
                if torch.cuda.can_device_access_peer(device.index, d):
                    torch.empty(1, device=f"cuda:{d}").to(device)
            except Exception:
                pass


class SymmetricHeap:
    """`nbytes` of data per rank, mapped on all ranks of `group` (None = single rank)."""

    def __init__(self, nbytes: int, group=None, device=None, backend: str = "auto"):
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.device = torch.device(device) if device is not None else \
            torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (nbytes + 255) // 256 * 256
        total = _FLAG_BYTES + self.nbytes
        self.backend = None
        self.multicast_ptr = 0
        self._keep = []
        if self.world == 1:
            self.local = torch.zeros(total, dtype=torch.uint8, device=self.device)
            self.peer_ptrs = [self.local.data_ptr()]
            self.backend = "local"
        else:
            ok = False
            if backend in ("auto", "symm_mem"):
                ok = self._init_symm_mem(total)
            if not ok and backend in ("auto", "ipc"):
                ok = self._init_ipc(total)
            if not ok:
                raise RuntimeError("could not create a symmetric heap (neither symmetric memory nor CUDA IPC)")
        self.flags = self.local[:_FLAG_BYTES].view(torch.int32)
        self.data = self.local[_FLAG_BYTES:]
        self._cursor = 0
        self._flag_cursor = 0
        self.epoch = 0

    # ------------------------------------------------------------------ set-up paths
    def _init_symm_mem(self, total):
        try:
            import torch.distributed._symmetric_memory as symm_mem

            t = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
            t.zero_()
            name = self.group.group_name if hasattr(self.group, "group_name") else self.group
            hdl = symm_mem.rendezvous(t, name)
            self.local = t
            self.peer_ptrs = [int(p) for p in hdl.buffer_ptrs]
            try:
                self.multicast_ptr = int(hdl.multicast_ptr or 0)
            except Exception:
                self.multicast_ptr = 0
            self._keep.append(hdl)
            self.backend = "symm_mem"
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
            return True
        except Exception as e:  # noqa: BLE001
            self._symm_error = repr(e)
            return False

    def _init_ipc(self, total):
        try:
            _enable_peer_access(self.device, self.world)
            # a dedicated allocation (not a slice of a cached segment) keeps offsets trivial
            t = torch.zeros(total, dtype=torch.uint8, device=self.device)
            handle = t.untyped_storage()._share_cuda_()
            gathered = [None] * self.world
            dist.all_gather_object(gathered, handle, group=self.group)
            ptrs = []
            for r, h in enumerate(gathered):
                if r == self.rank:
                    ptrs.append(t.data_ptr())
                    continue
                storage = torch.UntypedStorage._new_shared_cuda(*h)
                self._keep.append(storage)
                ptrs.append(storage.data_ptr())
            self.local = t
            self.peer_ptrs = ptrs
            self.backend = "ipc"
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
            return True
        except Exception as e:  # noqa: BLE001
            self._ipc_error = repr(e)
            return False

    # ------------------------------------------------------------------ sub-allocation
    def alloc(self, nbytes: int, align: int = 256):
        """Reserve `nbytes` at the same offset on every rank. Returns the data offset."""
        off = (self._cursor + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted ({off + nbytes} > {self.nbytes})")
        self._cursor = off + nbytes
        return off

    def alloc_flags(self, n: int):
        """Reserve `n` int32 flag words (same index on every rank). Returns the first index."""
        if self._flag_cursor + n > FLAG_WORDS:
            raise MemoryError("symmetric flag words exhausted")
        i = self._flag_cursor
        self._flag_cursor += n
        return i

    def tensor(self, offset: int, shape, dtype):
        n = int(torch.empty(0, dtype=dtype).element_size())
        numel = 1
        for s in shape:
            numel *= s
        return self.data[offset:offset + numel * n].view(dtype).view(*shape)

    def data_ptr(self, rank: int, offset: int = 0) -> int:
        return self.peer_ptrs[rank] + _FLAG_BYTES + offset

    def flag_ptr(self, rank: int, index: int) -> int:
        return self.peer_ptrs[rank] + 4 * index

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch
