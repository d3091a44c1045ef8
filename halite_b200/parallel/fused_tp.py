"""Fused compute + collective operators over symmetric memory.

`FusedAllGatherGemm`   y = all_gather(x_shard) @ W^T : a few CTAs of the GEMM launch pull the
                       peers' shards over NVLink into local staging while the tensor-core CTAs
                       start on the local shard; tiles wait only for the rows they read.
`FusedGemmReduceScatter` out_shard = reduce_scatter(x @ W^T): the epilogue stores every tile
                       straight into its owner's memory, then the same launch waits for the
                       peers' partials and reduces the own shard.

They replace the NCCL all-gather + cuBLAS and cuBLAS + NCCL reduce-scatter pairs of the
reference's tensor-parallel layers (transformers/attention.py:249-259,
transformers/feedforward.py:162-172) and of its micro-pipelined async-TP
(transformers/parallelize.py:133-142).

Synchronisation is by epoch-valued flag words in the symmetric heap, written with
system-scope release stores and read with bounded acquire spins; a wait that runs out records
a status code (see `ops.check_status`) and the launch still terminates.
"""

from __future__ import annotations

import torch

import halite_b200.ops as ops
from halite_b200.ops.linear import gemm
from halite_b200.parallel.symm import SymmetricHeap

_TILE_ROWS = 128


class FusedAllGatherGemm:
    def __init__(self, heap: SymmetricHeap, rows_per_rank: int, k: int, n_copy_ctas: int = 16,
                 buffers: int = 2):
        assert rows_per_rank % _TILE_ROWS == 0, "rows per rank must be a multiple of the 128-row tile"
        self.heap = heap
        self.world, self.rank = heap.world, heap.rank
        self.rows, self.k = rows_per_rank, k
        self.n_copy_ctas = n_copy_ctas if self.world > 1 else 0
        self.chunk_bytes = rows_per_rank * k * 2
        self.granule_bytes = _TILE_ROWS * k * 2
        self.n_buf = buffers
        self.offsets = [heap.alloc(self.chunk_bytes * self.world) for _ in range(buffers)]
        self.f_ready = [heap.alloc_flags(self.world) for _ in range(buffers)]
        self.f_done = [heap.alloc_flags(self.world) for _ in range(buffers)]
        dev = heap.device
        n_gran = self.world * rows_per_rank // _TILE_ROWS
        self.gran_flags = [torch.zeros(n_gran, dtype=torch.int32, device=dev) for _ in range(buffers)]
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.call = 0
        self.last_epoch = [0] * buffers

    def _buf(self):
        return self.call % self.n_buf

    def staging(self, buf=None):
        b = self._buf() if buf is None else buf
        return self.heap.tensor(self.offsets[b], (self.world * self.rows, self.k), torch.bfloat16)

    def input_slot(self):
        """Where the caller writes this rank's shard for the NEXT call (a view of the staging
        buffer). Blocks the stream until every peer has finished reading the slot's previous
        contents."""
        b = self._buf()
        if self.world > 1 and self.last_epoch[b] > 0:
            flags = self.heap.flags[self.f_done[b]:self.f_done[b] + self.world]
            ops.ext().wait_flags(flags, self.last_epoch[b], ops.status_word(self.heap.device))
        return self.staging(b)[self.rank * self.rows:(self.rank + 1) * self.rows]

    def __call__(self, weight, out=None, x_shard=None, b_mn=False):
        """weight: [N, K] bf16 (this rank's column shard), or [K, N] with b_mn. Returns
        [world * rows, N]."""
        b = self._buf()
        if x_shard is not None:
            self.input_slot().copy_(x_shard.reshape(self.rows, self.k))
        heap, w, r = self.heap, self.world, self.rank
        epoch = heap.next_epoch()
        staging = self.staging(b)
        gather = None
        if w > 1:
            # tell every peer (and myself, for the done accounting) that my shard is in place
            ptrs = [heap.flag_ptr(p, self.f_ready[b] + r) for p in range(w)]
            ptrs.append(heap.flag_ptr(r, self.f_done[b] + r))
            ops.ext().signal_flags(ptrs, epoch)
            gather = dict(
                src_ptrs=[0 if c == r else heap.data_ptr(c, self.offsets[b] + c * self.chunk_bytes)
                          for c in range(w)],
                peer_done_ptrs=[0 if c == r else heap.flag_ptr(c, self.f_done[b] + r) for c in range(w)],
                dst_ptr=staging.data_ptr(), chunk_bytes=self.chunk_bytes,
                granule_bytes=self.granule_bytes, n_copy_ctas=self.n_copy_ctas,
                flags_ptr=self.gran_flags[b].data_ptr(),
                ready_ptr=heap.flag_ptr(r, self.f_ready[b]), done_counter_ptr=self.counter.data_ptr(),
                epoch=epoch, dep=1, dep_row_bytes=self.k * 2, dep_base_offset=0,
                m_rot=r * self.rows // _TILE_ROWS, first_chunk=r)
        y = gemm(staging, weight, out=out, gather=gather, b_mn=b_mn)
        self.last_epoch[b] = epoch
        self.call += 1
        return y


class FusedGemmReduceScatter:
    def __init__(self, heap: SymmetricHeap, rows_per_rank: int, n: int, buffers: int = 2):
        assert n % 8 == 0
        self.heap = heap
        self.world, self.rank = heap.world, heap.rank
        self.rows, self.n = rows_per_rank, n
        self.slot_bytes = rows_per_rank * n * 2
        self.n_buf = buffers
        # recv[b][p]: this rank's chunk as computed by rank p
        self.recv_off = [heap.alloc(self.slot_bytes * self.world) for _ in range(buffers)]
        self.f_flags = [heap.alloc_flags(self.world) for _ in range(buffers)]
        dev = heap.device
        self.partial = torch.empty(rows_per_rank, n, dtype=torch.bfloat16, device=dev)
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.call = 0

    def __call__(self, x, weight, out=None, b_mn=False):
        """x: [world * rows, K_local], weight: [N, K_local] (or [K_local, N] with b_mn). Returns
        this rank's reduced [rows, N] shard of x @ weight^T summed over ranks."""
        heap, w, r = self.heap, self.world, self.rank
        b = self.call % self.n_buf
        epoch = heap.next_epoch()
        if out is None:
            out = torch.empty(self.rows, self.n, dtype=torch.bfloat16, device=x.device)
        if w == 1:
            gemm(x, weight, out=out, b_mn=b_mn)
            self.call += 1
            return out
        off = self.recv_off[b]
        scatter = dict(
            dst_ptrs=[self.partial.data_ptr() if c == r else heap.data_ptr(c, off + r * self.slot_bytes)
                      for c in range(w)],
            recv_ptrs=[0 if p == r else heap.data_ptr(r, off + p * self.slot_bytes) for p in range(w)],
            peer_flag_ptrs=[0 if c == r else heap.flag_ptr(c, self.f_flags[b] + r) for c in range(w)],
            my_flags_ptr=heap.flag_ptr(r, self.f_flags[b]), out_ptr=out.data_ptr(),
            cta_counter_ptr=self.counter.data_ptr(), rows_per_chunk=self.rows, rank=r, epoch=epoch,
            # start on the next rank's rows: what has to cross NVLink is computed first and the
            # rank's own rows last
            m_rot=((r + 1) % w) * self.rows // _TILE_ROWS if self.rows % _TILE_ROWS == 0 else 0)
        # the [M, N] `out` argument of the plain GEMM is unused in scatter mode: pass the partial
        gemm(x, weight, out=self.partial, scatter=scatter, b_mn=b_mn)
        self.call += 1
        return out
