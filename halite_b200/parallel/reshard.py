"""Fused trainer -> engine weight reshard (FSDP shards -> tensor-parallel inference layout).

`FusedResharder` walks the engine model's state dict once, finds every tensor inside the flat
unit buffers of the sharded training model, and records where each destination byte comes from:
which unit, which byte range of the unit's flat buffer, and, for a tensor-parallel engine, which
rows (column-parallel projections, also the separately cut q | k | v and gate | up blocks of packed
matrices) or which columns (row-parallel projections) this rank keeps. `run()` then fills all
engine tensors with ONE kernel launch (`csrc/reshard.cu`).

Where the bytes are read from depends on the training schedule:

* parameters kept gathered (the default): every rank already holds the whole flat buffer, so the
  kernel reads local memory only and the hand-over is a layout change;
* memory-lean schedule (`reshard_after_forward=True`): a rank holds only its shard. The shards
  are then placed in one symmetric heap (`place_shards_in_symmetric_memory`) and the kernel pulls
  each vector from the owning rank over NVLink with a plain load. No all-gather and no full
  tensor is materialised on the way.

Reference behaviour: distributed/state_dict.py:5-38 (per-tensor `full_tensor()` then copy),
infer/engine/model_runner.py:108-115.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

_COLS = 14       # int64 words of one segment: dst, src_base[8], src_byte0, src_pitch, shard_bytes, row_bytes, rows


def place_shards_in_symmetric_memory(state):
    """Move the `local_shard` of every resharding unit into one symmetric heap over the shard
    group, so peers can read it directly. Returns the heap (kept alive on `state`)."""
    from halite_b200.parallel.symm import SymmetricHeap

    units = [u for u in state.units if u.reshard]
    if not units:
        return None
    for u in units:
        u.param_shard()                      # makes sure the shard exists and is current
    sizes = [(u.shard_numel * u.local_shard.element_size() + 255) // 256 * 256 for u in units]
    heap = SymmetricHeap(sum(sizes) + 256 * len(units), group=state.shard_group, device=units[0].device)
    for u, nbytes in zip(units, sizes):
        off = heap.alloc(nbytes)
        buf = heap.tensor(off, (u.shard_numel,), u.local_shard.dtype)
        buf.copy_(u.local_shard)
        u.local_shard = buf
        u._heap_offset = off
    state.shard_heap = heap
    torch.cuda.synchronize(units[0].device)
    dist.barrier(state.shard_group)
    return heap


class FusedResharder:
    def __init__(self, train_model, target_state, tp_rank=0, tp_size=1, tp_plan=None):
        """`target_state`: {key: tensor} of the engine (allocated on the device, contiguous);
        `tp_plan`: {key: ("shard", dim) | ("shard_parts", dim, parts)} for the tensors of which
        the engine holds a 1 / tp_size slice."""
        state = train_model._hb_fsdp
        self.state = state
        self.group = state.shard_group
        where = {}
        for u in state.units:
            for m, n, _, off, numel in u.entries:
                where[id(m._parameters[n])] = (u, off)
        names = {}
        for name, p in train_model.named_parameters(remove_duplicate=False):
            names[name.replace("_orig_mod.", "")] = p
        self.rows = []
        self.fallback = []       # (key, target) pairs the kernel cannot express (odd sizes)
        tp_plan = tp_plan or {}
        for key, dst in target_state.items():
            p = names.get(key.replace("_orig_mod.", ""))
            if p is None or id(p) not in where or not dst.is_cuda:
                if p is None:
                    raise KeyError(f"the training model has no parameter {key!r}")
                self.fallback.append((key, dst, p))
                continue
            u, off = where[id(p)]
            es = p.element_size()
            shape = tuple(p.shape)
            rows_full = shape[0] if len(shape) > 1 else 1
            cols = p.numel() // rows_full
            plan = tp_plan.get(key) if tp_size > 1 else None
            segs = []           # (first element of the flat buffer, rows, row elements, pitch elements)
            if plan is None:
                segs.append((off, 1, p.numel(), p.numel()))
            elif plan[1] == 0:
                parts = plan[2] if plan[0] == "shard_parts" else [rows_full]
                at = 0
                for n in parts:
                    step = n // tp_size
                    segs.append((off + (at + tp_rank * step) * cols, 1, step * cols, step * cols))
                    at += n
            else:
                step = cols // tp_size
                segs.append((off + tp_rank * step, rows_full, step, cols))
            want = sum(r * n for _, r, n, _ in segs)
            ok = dst.is_contiguous() and dst.numel() == want and dst.dtype == p.dtype and dst.data_ptr() % 16 == 0 \
                and all((e0 * es) % 16 == 0 and (n * es) % 16 == 0 and (pitch * es) % 16 == 0 for e0, _, n, pitch in segs)
            if not ok:
                self.fallback.append((key, dst, p))
                continue
            at_bytes = 0
            for e0, r, n, pitch in segs:
                self.rows.append((u, dst.data_ptr() + at_bytes, e0 * es, pitch * es, n * es, r))
                at_bytes += r * n * es
        self.tp = (tp_rank, tp_size, tp_plan)
        self._table = None
        self._table_key = None

    def _build_table(self):
        device = self.state.units[0].device
        rows = []
        key = []
        for u, dst, src0, pitch, row_bytes, n_rows in self.rows:
            es = u.full_param.element_size()
            if u.reshard:
                heap = getattr(self.state, "shard_heap", None)
                if heap is None or not hasattr(u, "_heap_offset"):
                    raise RuntimeError("resharded units need place_shards_in_symmetric_memory() before a fused reshard")
                bases = [heap.data_ptr(r, u._heap_offset) for r in range(u.ws)]
                shard_bytes = u.shard_numel * es
            else:
                u.wait_gather()
                bases = [u.full_param.data_ptr()]
                shard_bytes = u.padded * es
            bases = bases + [0] * (8 - len(bases))
            rows.append([dst] + bases + [src0, pitch, shard_bytes, row_bytes, n_rows])
            key.append(bases[0])
        key = tuple(key)
        if self._table is None or self._table_key != key:
            self._table = torch.tensor(rows, dtype=torch.int64).to(device)
            self._table_key = key
        return self._table

    @torch.no_grad()
    def run(self):
        """Fill every engine tensor. With shards in peer memory the ranks meet before (all
        optimizer updates are in place) and after (nobody overwrites a shard that is still being
        read); both meetings are stream-ordered collectives, not host waits."""
        from halite_b200 import ops

        remote = any(u.reshard and u.ws > 1 for u, *_ in self.rows)
        if remote:
            self._sync()
        if self.rows:
            ops.ext().reshard_copy(self._build_table())
        for key, dst, p in self.fallback:
            self._slow_copy(key, dst, p)
        if remote:
            self._sync()

    def _sync(self):
        t = torch.zeros(1, device=self.state.units[0].device)
        dist.all_reduce(t, group=self.group)

    def _slow_copy(self, key, dst, p):
        from halite_b200.distributed.state_dict import reshard_state_dict

        self.state.wait_parameters()
        rank, size, plan = self.tp
        out = reshard_state_dict({key: p.detach()}, {key: dst}, tp_rank=rank, tp_size=size, tp_plan=plan, in_place=True)
        return out
