"""Sharded data parallelism on flat per-block buffers (the job FSDP2 does in the reference,
parallel/fsdp.py:8-60), laid out for a 180 GB GPU.

Each unit (one transformer block; the head unit: final norm + head; the root remainder: the
embedding and anything else) owns

* `full_param`  low-precision (bf16) flat buffer holding every parameter of the unit; the
                module's `nn.Parameter`s are views into it, so linears that read the same
                input (q|k|v, up|gate) are contiguous and run as ONE GEMM;
* `full_grad`   reduce-dtype (fp32) flat buffer; wgrad GEMMs accumulate straight into views of
                it (`param._hb_grad`), other gradients are copied in after the unit's backward;
* `master`, `exp_avg`, `exp_avg_sq`: fp32 shards (1 / dp_shard of the unit) for the optimizer.

Step schedule: reduce-scatter of a unit's gradient is launched on the communication stream
the moment the unit's backward ends and overlaps the next unit's backward; after the fused
AdamW has rewritten the rank's bf16 shard inside `full_param`, one all-gather per unit is
issued in forward order and each forward waits only for its own unit. Parameters stay
gathered between forward and backward (no second all-gather): 2 bytes / parameter of HBM
buys one collective per step instead of two. The AdamW kernels and the gathers are issued unit
by unit in the order the next forward uses the units, so that forward waits for the embedding's
gather only and every other gather hides under compute.

`reshard_after_forward=True` selects the memory-lean (ZeRO-3) schedule instead: a rank keeps only
its own bf16 shard of every unit (`local_shard`); a unit's `full_param` storage is allocated and
gathered right before the unit's forward (the next unit's gather is started at the same time),
released after it, gathered again before the unit's backward and released after it; the fp32
`full_grad` storage exists from the unit's backward until its reduce-scatter has finished. The
buffers are resized in place, so parameter and gradient views stay valid throughout.

With dp_replicate > 1 (HSDP) gradient shards are additionally all-reduced across replicas;
with dp_shard == 1 (DDP) a unit's "shard" is the whole buffer.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist
from torch import nn

from halite_b200.parallel import comm

_ALIGN = 128  # elements: keeps every shard 256-byte aligned in bf16 and 512 in fp32


class _UnitBoundary(torch.autograd.Function):
    """Identity placed on a unit's input: its backward runs after every gradient inside the
    unit has been produced."""

    @staticmethod
    def forward(ctx, x, unit):
        ctx.unit = unit
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.unit.post_backward()
        return g, None


class _UnitPreBackward(torch.autograd.Function):
    """Identity placed on a unit's output: its backward runs before any gradient inside the unit
    is computed (used to gather a resharded unit's parameters again)."""

    @staticmethod
    def forward(ctx, x, unit):
        ctx.unit = unit
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.unit.pre_backward()
        return g, None


def _free_storage(t):
    t.untyped_storage().resize_(0)


def _alloc_storage(t, numel):
    t.untyped_storage().resize_(numel * t.element_size())


class FlatUnit:
    def __init__(self, name, module_params, shard_group, replicate_group, param_dtype, reduce_dtype,
                 device, comm_stream=None):
        self.name = name
        self.shard_group = shard_group
        self.replicate_group = replicate_group
        self.ws = dist.get_world_size(shard_group) if shard_group is not None else 1
        self.rank = dist.get_rank(shard_group) if shard_group is not None else 0
        self.param_dtype = param_dtype
        self.reduce_dtype = reduce_dtype
        self.device = torch.device(device)
        self.comm_stream = comm_stream
        # decay parameters first, then no-decay (ndim < 2), so weight decay is a range split
        decay = [(m, n, p) for (m, n, p) in module_params if p.ndim >= 2]
        no_decay = [(m, n, p) for (m, n, p) in module_params if p.ndim < 2]
        self.entries = []   # (module, attr name, param, offset, numel)
        off = 0
        for group in (decay, no_decay):
            for m, n, p in group:
                off = (off + 7) // 8 * 8          # 16-byte aligned starts (TMA bases)
                self.entries.append((m, n, p, off, p.numel()))
                off += p.numel()
            if group is decay:
                self.decay_end = off
        self.numel = off
        # padding to a multiple of 8192 as well makes the flat length the same for every
        # power-of-two shard count up to 64, so optimizer shards reshard without translation
        chunk = math.lcm(self.ws * _ALIGN, 8192)
        self.padded = max(chunk, (off + chunk - 1) // chunk * chunk)
        self.shard_numel = self.padded // self.ws
        self.lo = self.rank * self.shard_numel
        self.hi = self.lo + self.shard_numel

        self.full_param = torch.zeros(self.padded, dtype=param_dtype, device=self.device)
        self.full_grad = torch.zeros(self.padded, dtype=reduce_dtype, device=self.device)
        self.grad_shard = (self.full_grad if self.ws == 1
                           else torch.zeros(self.shard_numel, dtype=reduce_dtype, device=self.device))
        self.master = None        # fp32 shard, created by `init_master`
        self._written = set()
        self._gather_event = None
        self._reduce_event = None
        self._reduce_work = None
        self._gather_work = None
        self._backward_done = False
        self._needs_reduce = False
        self.defer_reduce = False  # set by `ShardedModel.no_sync()`: backward passes only accumulate
        # memory-lean schedule (`enable_reshard`): the rank's own shard lives in `local_shard`, the
        # full buffers are only allocated around the unit's forward / backward
        self.reshard = False
        self.local_shard = None
        self.materialized = True      # `full_param` is allocated and current
        self.grad_allocated = True
        self.prev_unit = None         # neighbours in forward order (prefetch targets)
        self.next_unit = None
        self.state = None             # the owning ShardedModel
        self.fused = None         # FusedGather state once `enable_fused_gather` has run
        self.fused_reduce = None  # FusedReduce state once `enable_fused_reduce` has run
        self._adopt_params()

    # ------------------------------------------------------------------ parameter views
    def _adopt_params(self):
        for m, n, p, off, numel in self.entries:
            view = self.full_param[off:off + numel].view(p.shape)
            if p.device.type != "meta":
                view.copy_(p.detach().to(view.dtype))
            new_p = nn.Parameter(view, requires_grad=p.requires_grad)
            new_p._hb_grad = self.full_grad[off:off + numel].view(p.shape)
            new_p._hb_grad_owner = self
            new_p._hb_unit_range = (off, numel)
            if hasattr(p, "_hb_tp_replicated"):
                new_p._hb_tp_replicated = p._hb_tp_replicated
            # keep initialiser-visible attributes
            m._parameters[n] = new_p

    def rehome(self, buffer):
        """Move `full_param` into `buffer` (same length and dtype, e.g. symmetric memory): values
        are copied and every parameter keeps its identity, only its storage changes."""
        buffer.copy_(self.full_param)
        self.full_param = buffer
        for m, n, _, off, numel in self.entries:
            p = m._parameters[n]
            p.data = buffer[off:off + numel].view(p.shape)

    def rehome_grad(self, buffer):
        """Move `full_grad` into `buffer` (fp32, same length); every parameter's main-grad view
        follows."""
        buffer.copy_(self.full_grad)
        self.full_grad = buffer
        for m, n, _, off, numel in self.entries:
            p = m._parameters[n]
            p._hb_grad = buffer[off:off + numel].view(p.shape)

    def params(self):
        return [m._parameters[n] for m, n, _, _, _ in self.entries]

    def named_views(self):
        """[(module, name, offset, numel, shape)] for checkpointing and resharding."""
        return [(m, n, off, numel, m._parameters[n].shape) for m, n, _, off, numel in self.entries]

    def fused_view(self, module, names):
        """One [sum(out_features), in_features] view over consecutive linear weights, or None
        when they are not adjacent in the flat buffer."""
        found = []
        for sub in names:
            lin = getattr(module, sub)
            if getattr(lin, "bias", None) is not None:
                return None
            hit = [(off, numel, m._parameters[n]) for m, n, _, off, numel in self.entries
                   if m is lin and n == "weight"]
            if not hit:
                return None
            found.append(hit[0])
        start = found[0][0]
        cur = start
        cols = found[0][2].shape[1]
        rows = 0
        for off, numel, p in found:
            if off != cur or p.shape[1] != cols:
                return None
            cur += numel
            rows += p.shape[0]
        w = self.full_param[start:cur].view(rows, cols)
        # a leaf that "requires grad" so autograd always visits the wgrad; the gradient
        # itself goes to the flat buffer through the main-grad protocol
        w.requires_grad_(any(p.requires_grad for _, _, p in found))
        w._hb_grad = self.full_grad[start:cur].view(rows, cols)
        w._hb_grad_owner = self
        w._hb_members = tuple(p for _, _, p in found)
        return w

    # ------------------------------------------------------------------ gradient bookkeeping
    def mark_written(self, param) -> bool:
        """Called by a wgrad that is about to write `param._hb_grad`; returns True when the
        buffer already holds this step's partial sum (so the GEMM must accumulate)."""
        members = getattr(param, "_hb_members", None) or (param,)
        acc = all(id(p) in self._written for p in members)
        if not acc and any(id(p) in self._written for p in members):
            # mixed state (one member written separately): cannot overwrite; caller accumulates
            # after we zero the unwritten members
            for p in members:
                if id(p) not in self._written:
                    p._hb_grad.zero_()
            acc = True
        for p in members:
            self._written.add(id(p))
        return acc

    # ------------------------------------------------------------------ memory-lean schedule
    def enable_reshard(self):
        if self.ws > 1:
            self.reshard = True

    def materialize(self, prefetch=None):
        """Allocate `full_param` and gather it from the ranks' `local_shard`s (on the communication
        stream when there is one). `prefetch` names a neighbour whose gather is started as well."""
        if self.reshard and not self.materialized:
            # The gather rewrites the buffer with the values it held when autograd saved views of
            # it in the forward pass, so the saved tensors stay valid: keep the version counter.
            with torch.autograd._unsafe_preserve_version_counter(self.full_param):
                if self.device.type == "cuda" and self.comm_stream is not None:
                    _alloc_storage(self.full_param, self.padded)     # on the compute stream: it frees it later
                    ev = torch.cuda.Event()
                    ev.record()
                    with torch.cuda.stream(self.comm_stream):
                        self.comm_stream.wait_event(ev)
                        comm.all_gather_flat(self.full_param, self.local_shard, self.shard_group)
                        self._gather_event = torch.cuda.Event()
                        self._gather_event.record()
                else:
                    _alloc_storage(self.full_param, self.padded)
                    comm.all_gather_flat(self.full_param, self.local_shard, self.shard_group)
            self.materialized = True
        if prefetch is not None:
            prefetch.materialize()

    def release(self):
        """Keep only this rank's shard of the parameters."""
        if not self.reshard or not self.materialized:
            return
        self.wait_gather()
        if self.local_shard is None:
            self.local_shard = self.full_param[self.lo:self.hi].clone()
        else:
            # in-place edits made while the unit was whole (initialisation, a loaded checkpoint)
            self.local_shard.copy_(self.full_param[self.lo:self.hi])
        _free_storage(self.full_param)
        self.materialized = False

    def ensure_grad(self):
        if not self.grad_allocated:
            _alloc_storage(self.full_grad, self.padded)
            self.full_grad.zero_()      # padding and alignment gaps take part in the reduction and the norm
            self.grad_allocated = True

    def release_grad(self):
        """Free `full_grad` once its reduction has finished (the current stream waits for it)."""
        if not self.reshard or not self.grad_allocated or self._needs_reduce:
            return
        if self._reduce_event is not None:
            torch.cuda.current_stream().wait_event(self._reduce_event)
        _free_storage(self.full_grad)
        self.grad_allocated = False

    def pre_backward(self):
        if self.reshard:
            self.materialize(prefetch=self.prev_unit)
            self.wait_gather()
            self.ensure_grad()

    def post_forward(self):
        if self.reshard:
            self.release()

    def pre_forward(self):
        if self.reshard:
            self.materialize(prefetch=self.next_unit)
        self.wait_gather()
        # the backward pass that follows writes gradients: an earlier micro-batch's reduction of
        # this unit must have finished with the buffer (the wait is queued on the stream now, the
        # reduction itself is long done by the time backward reaches the unit)
        self.wait_reduce_before_write()
        if self.fused is not None and self.fused.pending:
            # nobody carried this unit's gather (first block, or the carrying GEMM did not run)
            self.fused.run_standalone()
        self._backward_done = False

    def wait_gather(self):
        if self._gather_event is not None:
            torch.cuda.current_stream().wait_event(self._gather_event)
            self._gather_event = None
        if self._gather_work is not None:
            self._gather_work.wait()
            self._gather_work = None

    def post_backward(self):
        """Collect stray `.grad`s, zero what was not written, start the gradient reduction."""
        if self._backward_done:
            return
        self._backward_done = True
        self.ensure_grad()          # (a unit whose output needed no gradient never saw `pre_backward`)
        # a reduction of an earlier pass may still be reading (or, when the shard is the whole
        # buffer, rewriting) the gradient buffer this pass has just added to
        self.wait_reduce_before_write()
        for m, n, _, off, numel in self.entries:
            p = m._parameters[n]
            if p.grad is not None:
                if id(p) in self._written:
                    p._hb_grad.add_(p.grad.to(self.reduce_dtype))
                else:
                    p._hb_grad.copy_(p.grad)
                    self._written.add(id(p))
                p.grad = None
            elif id(p) not in self._written:
                p._hb_grad.zero_()
                self._written.add(id(p))
        # `_written` stays set until the optimizer has consumed the gradients (or `zero_grad`):
        # a further backward pass of the same step (micro-batches) accumulates into the buffer and
        # the reduction below then runs again on the running sum
        # parameters replicated over tensor-parallel ranks saw only this rank's token shard
        for m, n, _, off, numel in self.entries:
            p = m._parameters[n]
            tp = getattr(p, "_hb_tp_replicated", None)
            if tp is not None and tp.size > 1:
                dist.all_reduce(p._hb_grad, group=tp.group)
        if self.defer_reduce:
            self._needs_reduce = True
        else:
            self.start_reduce()
        if self.reshard:
            self.release()
            if self.state is not None:
                self.state.grad_released_later(self)

    def wait_reduce_before_write(self):
        """Order the current stream after a reduction of this unit that is still in flight."""
        if self._reduce_event is not None:
            torch.cuda.current_stream().wait_event(self._reduce_event)

    def start_reduce(self):
        self._needs_reduce = False
        if self.ws == 1 and self.replicate_group is None:
            return
        if self.fused_reduce is not None:
            self.fused_reduce.publish()
            return
        if self.device.type == "cuda" and self.comm_stream is not None:
            ev = torch.cuda.Event()
            ev.record()
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ev)
                self._reduce()
                self._reduce_event = torch.cuda.Event()
                self._reduce_event.record()
        else:
            self._reduce()

    def _reduce(self):
        if self.ws > 1:
            comm.reduce_scatter_flat(self.grad_shard, self.full_grad, self.shard_group, average=True)
        if self.replicate_group is not None:
            comm.all_reduce(self.grad_shard, self.replicate_group, average=True)

    def wait_reduce(self):
        if self.fused_reduce is not None and self.fused_reduce.pending:
            self.fused_reduce.run_standalone()       # nobody carried it (last unit of the backward pass)
        if self._reduce_event is not None:
            torch.cuda.current_stream().wait_event(self._reduce_event)
            self._reduce_event = None

    # ------------------------------------------------------------------ optimizer side
    def init_master(self):
        """fp32 master copy of this rank's shard, taken from the current low-precision values."""
        self.master = self.param_shard().float().clone()
        return self.master

    def param_shard(self):
        """This rank's low-precision shard (what the optimizer rewrites). On the memory-lean
        schedule that is `local_shard`; a unit that is whole at this point is released first, so
        its current values are carried over."""
        if self.reshard:
            self.release()
            return self.local_shard
        return self.full_param[self.lo:self.hi]

    def decay_split(self):
        """Element ranges of this rank's shard with / without weight decay:
        ((lo, hi) decay, (lo, hi) no-decay) in shard coordinates."""
        d_hi = min(max(self.decay_end - self.lo, 0), self.shard_numel)
        return (0, d_hi), (d_hi, self.shard_numel)

    def start_gather(self, epoch=None):
        """Make the updated shards visible everywhere: an all-gather into `full_param` (in place)
        on the comm stream, or, with the fused path, a flag that lets the peers' copy CTAs pull
        this rank's shard from inside one of their GEMM launches."""
        if self.ws == 1:
            return
        if self.reshard:
            return          # gathered lazily, right before the unit's next forward
        if self.fused is not None and epoch is not None:
            self.fused.publish(epoch)
            return
        if self.device.type == "cuda" and self.comm_stream is not None:
            ev = torch.cuda.Event()
            ev.record()
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ev)
                comm.all_gather_flat(self.full_param, self.param_shard(), self.shard_group)
                self._gather_event = torch.cuda.Event()
                self._gather_event.record()
        else:
            comm.all_gather_flat(self.full_param, self.param_shard(), self.shard_group)

    def sync_from_rank_shards(self):
        """Make `full_param` identical everywhere (used once after initialisation)."""
        if self.reshard and not self.materialized:
            self.materialize()
            self.wait_gather()
        if self.ws > 1:
            comm.all_gather_flat(self.full_param, self.full_param[self.lo:self.hi].clone(), self.shard_group)
        if self.replicate_group is not None:
            dist.broadcast(self.full_param, src=dist.get_global_rank(self.replicate_group, 0),
                           group=self.replicate_group)


class FusedGather:
    """All-gather of one unit's parameters carried by a GEMM launch: a few CTAs of that launch
    copy the peers' shards out of their symmetric-memory `full_param` into the local one with
    plain loads over NVLink while the other CTAs compute (`GatherParams` of the GEMM kernel).

    Protocol per optimizer step (epoch = step number, flags only ever grow):
      owner   after AdamW rewrote its shard: writes `ready[owner]` = epoch on every peer
      reader  copy CTAs wait for `ready[c]` >= epoch before touching chunk c; when the last copy
              CTA is done it writes `done[reader]` = epoch on every owner
      owner   before the next AdamW overwrites the shard: waits for `done[r]` >= epoch of all r
    """

    GRANULE = 256 * 1024
    COPY_CTAS = 16

    def __init__(self, unit, heap, offset, f_ready, f_done):
        self.unit, self.heap, self.offset = unit, heap, offset
        self.f_ready, self.f_done = f_ready, f_done
        self.chunk_bytes = unit.shard_numel * unit.full_param.element_size()
        n_gran = unit.ws * ((self.chunk_bytes + self.GRANULE - 1) // self.GRANULE)
        self.gran_flags = torch.zeros(n_gran, dtype=torch.int32, device=unit.device)
        self.counter = torch.zeros(1, dtype=torch.int32, device=unit.device)
        self.pending = 0          # epoch whose gather has not been launched yet
        self.published = 0        # last epoch this rank announced
        self.launches = 0         # gathers carried by a model GEMM / launched on their own
        self.standalone = 0

    def publish(self, epoch):
        from halite_b200 import ops

        u, h = self.unit, self.heap
        ptrs = [h.flag_ptr(p, self.f_ready + u.rank) for p in range(u.ws) if p != u.rank]
        ptrs.append(h.flag_ptr(u.rank, self.f_done + u.rank))      # own slot of the reader accounting
        ops.ext().signal_flags(ptrs, epoch)
        self.pending = self.published = epoch

    def wait_readers(self):
        """Block the stream until every peer has read the shard announced last."""
        if self.published:
            from halite_b200 import ops

            flags = self.heap.flags[self.f_done:self.f_done + self.unit.ws]
            ops.ext().wait_flags(flags, self.published, ops.status_word(self.unit.device))

    def take(self):
        """Gather description for the GEMM that carries this unit's gather (None when there is
        nothing to fetch); hands the job over, so only one launch gets it."""
        if not self.pending:
            return None
        epoch, self.pending = self.pending, 0
        u, h = self.unit, self.heap
        self.launches += 1
        return dict(
            src_ptrs=[0 if c == u.rank else h.data_ptr(c, self.offset + c * self.chunk_bytes) for c in range(u.ws)],
            peer_done_ptrs=[0 if c == u.rank else h.flag_ptr(c, self.f_done + u.rank) for c in range(u.ws)],
            dst_ptr=u.full_param.data_ptr(), chunk_bytes=self.chunk_bytes, granule_bytes=self.GRANULE,
            n_copy_ctas=self.COPY_CTAS, flags_ptr=self.gran_flags.data_ptr(),
            ready_ptr=h.flag_ptr(u.rank, self.f_ready), done_counter_ptr=self.counter.data_ptr(),
            epoch=epoch, dep=0, dep_row_bytes=0, dep_base_offset=0, first_chunk=u.rank)

    def run_standalone(self):
        """The same copy CTAs under a one-tile GEMM on scratch operands."""
        from halite_b200.ops.linear import gemm

        gather = self.take()
        if gather is None:
            return
        self.standalone += 1
        a, b, out = _scratch_gemm_operands(self.unit.device)
        gemm(a, b, out=out, gather=gather)


class FusedReduce:
    """Reduce-scatter of one unit's fp32 gradients carried by a GEMM launch of the backward pass:
    a few CTAs of that launch read this rank's range out of every rank's symmetric-memory
    `full_grad` over NVLink (one `multimem.ld_reduce` per 16 bytes when the heap has an NVLS
    multicast mapping: the switch adds the ranks' copies; else one plain load per rank, added in
    rank order), scale by 1 / ranks and write the rank's `grad_shard`, while the other CTAs compute. Flags as in `FusedGather`:
    `ready[owner]` = epoch once a rank's gradients of the unit are complete, `done[reader]` =
    epoch once a rank has read everybody's range (the buffer may be overwritten after that)."""

    COPY_CTAS = 32

    def __init__(self, unit, heap, offset, f_ready, f_done):
        import os

        self.unit, self.heap, self.offset = unit, heap, offset
        self.f_ready, self.f_done = f_ready, f_done
        self.counter = torch.zeros(1, dtype=torch.int32, device=unit.device)
        # HB_FSDP_NVLS=0 keeps the plain peer loads (needed where a rank may leave while its memory
        # is bound to the multicast object, and on switches without in-network reduction)
        self.use_multimem = os.environ.get("HB_FSDP_NVLS", "1") != "0"
        self.epoch = 0
        self.pending = 0
        self.launches = 0
        self.standalone = 0

    def publish(self):
        from halite_b200 import ops

        u, h = self.unit, self.heap
        self.epoch += 1
        ptrs = [h.flag_ptr(p, self.f_ready + u.rank) for p in range(u.ws) if p != u.rank]
        ptrs.append(h.flag_ptr(u.rank, self.f_done + u.rank))
        ops.ext().signal_flags(ptrs, self.epoch)
        self.pending = self.epoch

    def wait_readers(self):
        """Block the stream until every peer has read this rank's gradients of the last pass."""
        if self.epoch:
            from halite_b200 import ops

            flags = self.heap.flags[self.f_done:self.f_done + self.unit.ws]
            ops.ext().wait_flags(flags, self.epoch, ops.status_word(self.unit.device))

    def take(self):
        if not self.pending:
            return None
        epoch, self.pending = self.pending, 0
        u, h = self.unit, self.heap
        self.launches += 1
        mine = self.offset + u.lo * 4      # this rank's range inside every rank's fp32 buffer
        extra = {}
        if h.multicast_ptr and self.use_multimem:
            # the heap is bound to an NVLink multicast object: the switch adds the ranks' copies
            from halite_b200.parallel.symm import _FLAG_BYTES

            extra["mc_src_ptr"] = h.multicast_ptr + _FLAG_BYTES + mine
        return dict(
            **extra,
            src_ptrs=[h.data_ptr(c, mine) for c in range(u.ws)],
            peer_done_ptrs=[0 if c == u.rank else h.flag_ptr(c, self.f_done + u.rank) for c in range(u.ws)],
            dst_ptr=0, chunk_bytes=16, granule_bytes=16, n_copy_ctas=self.COPY_CTAS, flags_ptr=0,
            ready_ptr=h.flag_ptr(u.rank, self.f_ready), done_counter_ptr=self.counter.data_ptr(),
            epoch=epoch, dep=0, dep_row_bytes=0, first_chunk=u.rank,
            reduce_out_ptr=u.grad_shard.data_ptr(), reduce_numel=u.shard_numel, reduce_scale=1.0 / u.ws)

    def run_standalone(self):
        from halite_b200.ops.linear import gemm

        gather = self.take()
        if gather is None:
            return
        self.standalone += 1
        a, b, out = _scratch_gemm_operands(self.unit.device)
        gemm(a, b, out=out, gather=gather)


_SCRATCH = {}


def _scratch_gemm_operands(device):
    """Operands of the one-tile GEMM that hosts copy CTAs when no model GEMM is at hand."""
    key = torch.device(device)
    if key not in _SCRATCH:
        _SCRATCH[key] = (torch.zeros(128, 64, dtype=torch.bfloat16, device=key),
                         torch.zeros(64, 64, dtype=torch.bfloat16, device=key),
                         torch.zeros(128, 64, dtype=torch.bfloat16, device=key))
    return _SCRATCH[key]


def enable_fused_reduce(state):
    """Move the block units' fp32 `full_grad` buffers into one symmetric-memory heap and replace
    their reduce-scatter collective by `FusedReduce`: the reduction of block i rides on the first
    backward GEMM of block i - 1; the first block's runs on its own when the backward pass ends.
    The root unit keeps the collective."""
    from halite_b200.parallel.symm import SymmetricHeap

    units = [u for u in state.units if u is not state.root_unit and u is not state.head_unit and u.ws > 1]
    if not units or units[0].device.type != "cuda" or state.replicate_group is not None \
            or units[0].reduce_dtype != torch.float32:
        return False
    sizes = [(u.padded * 4 + 255) // 256 * 256 for u in units]
    heap = SymmetricHeap(sum(sizes) + 256 * len(units), group=state.shard_group, device=units[0].device)
    state.reduce_heap = heap
    for u, nbytes in zip(units, sizes):
        off = heap.alloc(nbytes)
        u.rehome_grad(heap.tensor(off, (u.padded,), torch.float32))
        u.fused_reduce = FusedReduce(u, heap, off, heap.alloc_flags(u.ws), heap.alloc_flags(u.ws))
    _install_fused_views(state.model, state.units)
    for prev, nxt in zip(units[:-1], units[1:]):
        mats = [(m, n) for m, n, p, _, _ in prev.entries if p.ndim == 2 and isinstance(m, nn.Linear)]
        if mats:
            m, n = mats[-1]
            m._parameters[n]._hb_carry_bwd = nxt.fused_reduce.take
    torch.cuda.synchronize(units[0].device)
    dist.barrier(state.shard_group)
    return True


def enable_fused_gather(state, carried=True):
    """Move the block units' `full_param` buffers into one symmetric-memory heap and switch their
    post-optimizer all-gather to the GEMM-carried copy. The root unit (embedding, head, final
    norm: used before any GEMM of the step) keeps the collective. With `carried`, the gather of
    block i + 1 rides on the last GEMM of block i's forward; otherwise (and for the first block)
    it is launched on its own right before the block runs."""
    from halite_b200.parallel.symm import SymmetricHeap

    units = [u for u in state.units if u is not state.root_unit and u is not state.head_unit and u.ws > 1]
    if not units or units[0].device.type != "cuda":
        return False
    elem = units[0].full_param.element_size()
    sizes = [(u.padded * elem + 255) // 256 * 256 for u in units]
    heap = SymmetricHeap(sum(sizes) + 256 * len(units), group=state.shard_group, device=units[0].device)
    state.gather_heap = heap
    for u, nbytes in zip(units, sizes):
        off = heap.alloc(nbytes)
        u.rehome(heap.tensor(off, (u.padded,), u.full_param.dtype))
        u.fused = FusedGather(u, heap, off, heap.alloc_flags(u.ws), heap.alloc_flags(u.ws))
    _install_fused_views(state.model, state.units)
    if carried:
        for prev, nxt in zip(units[:-1], units[1:]):
            # last weight matrix of the previous block in module order (the down projection)
            mats = [(m, n) for m, n, p, _, _ in prev.entries if p.ndim == 2 and isinstance(m, nn.Linear)]
            if mats:
                m, n = mats[-1]
                m._parameters[n]._hb_carry = nxt.fused.take
    torch.cuda.synchronize(units[0].device)
    dist.barrier(state.shard_group)
    return True


class ShardedModel:
    """Book-keeping object attached to a wrapped model as `model._hb_fsdp`."""

    def __init__(self, model, units, root_unit, shard_group, replicate_group, comm_stream, head_unit=None):
        self.model = model
        self.units: list[FlatUnit] = units        # order of use in a forward pass: root, blocks, head
        self.root_unit = root_unit                # embedding and whatever no other unit took
        self.head_unit = head_unit                # final norm + head (None: they live in the root unit)
        self.shard_group = shard_group
        self.replicate_group = replicate_group
        self.comm_stream = comm_stream
        self.gather_heap = None
        self.reduce_heap = None
        self._grad_pending = []
        for a, b in zip(units[:-1], units[1:]):
            a.next_unit, b.prev_unit = b, a
        for u in units:
            u.state = self

    def wait_parameters(self):
        """Make the current stream see whole, current parameters in every unit: waits for the
        collective gathers in flight and launches the carried gathers nobody has carried yet.
        Anything that reads or writes parameters outside the model's own forward (state_dict,
        checkpoint staging, weight export to an engine, in-place re-normalisation) calls this."""
        for u in self.units:
            u.materialize()
            u.wait_gather()
        self.flush_gathers()

    def grad_released_later(self, unit):
        """A resharded unit's gradient buffer is freed when the NEXT unit finishes its backward:
        by then the reduction has had a whole unit's backward to complete, so the wait is free."""
        older, self._grad_pending = self._grad_pending, [unit]
        for u in older:
            if u is not unit:
                u.release_grad()

    def release_gradients(self):
        for u in self._grad_pending:
            u.release_grad()
        self._grad_pending = []

    def no_sync(self):
        """Context manager for gradient accumulation: backward passes inside it only add into the
        flat gradient buffers; the reduce-scatter / all-reduce of each unit is started by the
        first backward pass outside it (or by `finish_backward`), once per optimizer step."""
        state = self

        class _NoSync:
            def __enter__(self_inner):
                for u in state.units:
                    u.defer_reduce = True

            def __exit__(self_inner, *exc):
                for u in state.units:
                    u.defer_reduce = False
                return False

        return _NoSync()

    def flush_gathers(self):
        """Launch every gather that is still waiting for its carrier (before anything other than
        the model's own forward reads the parameters: state_dict, weight export, evaluation of a
        sub-module)."""
        for u in self.units:
            if u.fused is not None and u.fused.pending:
                u.fused.run_standalone()

    def finish_backward(self):
        """Run after `loss.backward()`: closes the root unit (and any unit whose boundary did
        not fire, e.g. one whose input needed no gradient)."""
        for u in self.units:
            u.post_backward()
            if u._needs_reduce:
                u.start_reduce()

    def wait_reductions(self):
        for u in self.units:
            u.wait_reduce()
        self.release_gradients()

    def sync_parameters(self):
        for u in self.units:
            u.sync_from_rank_shards()

    def refresh_fused_views(self):
        _install_fused_views(self.model, self.units)

    def all_group(self):
        return self.shard_group


def _install_fused_views(model, units):
    by_module = {}
    for u in units:
        for m, n, _, _, _ in u.entries:
            by_module[id(m)] = u
    for mod in model.modules():
        groups = getattr(mod, "fusable_linears", None)
        if groups is None:
            continue
        fused = {}
        for key, names in groups().items():
            lin = getattr(mod, names[0], None)
            u = by_module.get(id(lin))
            if u is None:
                continue
            w = u.fused_view(mod, names)
            if w is not None:
                fused[key] = w
        mod._hb_fused = fused


def _unit_params(module: nn.Module, exclude: set[int]):
    out = []
    seen = set()
    for m in module.modules():
        for n, p in m._parameters.items():
            if p is None or id(p) in exclude or id(p) in seen:
                continue
            seen.add(id(p))
            out.append((m, n, p))
    return out


def apply_fsdp(model, mesh=None, param_dtype=torch.bfloat16, reduce_dtype=torch.float32,
               reshard_after_forward=False, device=None, blocks_attr="blocks", force_fsdp=False,
               block_iterator=None, fused_all_gather=None, fused_reduce_scatter=None,
               tail_attrs=("post_blocks", "head")):
    """Shard `model` over the mesh's data-parallel dimensions. Returns the same module, with
    parameters re-homed into flat unit buffers and `model._hb_fsdp` set.

    `mesh` is a `ParallelDims` after `build_mesh()` (or None for a single process).
    `block_iterator(model)` may yield `(key, block, container)` for models whose blocks live in
    more than one container (an encoder's blocks followed by the model's own); each yielded block
    becomes a unit. Without it the units are the entries of `model.<blocks_attr>`.
    `tail_attrs` names the modules that run after the last block; when the model's forward calls
    the pre-block hook with index == number of blocks before them, they form the "head" unit.
    `fused_all_gather` (default: the HB_FSDP_FUSED_GATHER environment variable) replaces the block
    units' parameter all-gather collective by copies carried inside GEMM launches (`FusedGather`);
    `fused_reduce_scatter` (HB_FSDP_FUSED_REDUCE) does the same for the gradient reduce-scatter
    (`FusedReduce`).
    """
    shard_group = mesh.group("dp_shard") if mesh is not None else None
    replicate_group = mesh.group("dp_replicate") if mesh is not None else None
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
            else torch.device("cpu")
    device = torch.device(device)
    comm_stream = torch.cuda.Stream(device) if device.type == "cuda" else None
    if device.type == "cuda":
        # collectives will run beside the GEMMs and hold some SMs: let the GEMM hand its tiles
        # out through a counter so that clusters which start late take fewer tiles
        n_ranks = (dist.get_world_size(shard_group) if shard_group is not None else 1) * \
            (dist.get_world_size(replicate_group) if replicate_group is not None else 1)
        if n_ranks > 1:
            from halite_b200 import ops

            ops.ext().gemm_set_dynamic_schedule(True)

    units = []
    taken: set[int] = set()
    calls_block_hooks = hasattr(model, "block_hooks")     # the model's forward announces each block
    block_units = {}
    if block_iterator is not None:
        names = {id(m): n for n, m in model.named_modules()}
        listed = [(f"{names.get(id(container), blocks_attr)}.{key}", block, None)
                  for key, block, container in block_iterator(model)]
        calls_block_hooks = False
    else:
        blocks = getattr(model, blocks_attr, None)
        listed = [(f"{blocks_attr}.{key}", block, int(key)) for key, block in blocks.items()] \
            if blocks is not None else []
    for name, block, index in listed:
        ps = _unit_params(block, taken)
        if not ps:
            continue
        taken.update(id(p) for _, _, p in ps)
        u = FlatUnit(name, ps, shard_group, replicate_group, param_dtype, reduce_dtype, device, comm_stream)
        units.append(u)
        if index is not None:
            block_units[index] = u
        taken.update(id(p) for p in u.params())   # the re-homed Parameter objects
    # The output side of the model (final norm + head) becomes a unit of its own when the model's
    # forward announces it (hook index == number of blocks): its gradients are the first ones of
    # the backward pass, so their reduction starts at the top of backward and hides under all the
    # blocks, instead of waiting in the root unit until the pass is over; and its parameters are
    # the last ones the next forward needs, so its gather is queued last.
    head_unit = None
    tail_mods = [getattr(model, a, None) for a in tail_attrs]
    tied = getattr(model, "tie_embeds", False)
    if calls_block_hooks and block_units and not tied and tail_mods and tail_mods[-1] is not None:
        ps = []
        for mod in tail_mods:
            if mod is not None:
                got = _unit_params(mod, taken)
                taken.update(id(p) for _, _, p in got)
                ps.extend(got)
        if ps:
            head_unit = FlatUnit("head", ps, shard_group, replicate_group, param_dtype, reduce_dtype, device,
                                 comm_stream)
            taken.update(id(p) for p in head_unit.params())
            block_units[len(listed)] = head_unit
    # tied head/embedding weights are one parameter: `_unit_params` de-duplicates by identity
    root_ps = _unit_params(model, taken)
    root = FlatUnit("root", root_ps, shard_group, replicate_group, param_dtype, reduce_dtype, device,
                    comm_stream)
    # order of use in a forward pass: root (embedding), the blocks, the head
    units.insert(0, root)
    if head_unit is not None:
        units.append(head_unit)
    if tied and getattr(model, "head", None) is not None:
        model.head.tie_weight(model.embedding.embed_weight)

    # move remaining buffers
    for mod in model.modules():
        for n, b in list(mod._buffers.items()):
            if b is not None and b.device != device:
                mod._buffers[n] = torch.empty_like(b, device=device) if b.device.type == "meta" \
                    else b.to(device)

    state = ShardedModel(model, units, root, shard_group, replicate_group, comm_stream, head_unit)
    model._hb_fsdp = state
    _install_fused_views(model, units)

    def pre_block(i, x):
        u = block_units.get(i)
        if u is None:
            return x
        u.pre_forward()
        if torch.is_grad_enabled() and x.requires_grad:
            x = _UnitBoundary.apply(x, u)
        return x

    def post_block(i, x, residual=None):
        u = block_units.get(i)
        if u is None or not u.reshard:
            return x, residual
        if torch.is_grad_enabled():
            # whichever of the block's outputs receives its gradient first brings the unit back
            if x.requires_grad:
                x = _UnitPreBackward.apply(x, u)
            if residual is not None and residual.requires_grad:
                residual = _UnitPreBackward.apply(residual, u)
        u.post_forward()
        return x, residual

    model.block_hooks = (pre_block, post_block)

    def _to_param_dtype(value):
        if torch.is_tensor(value) and value.is_floating_point() and value.dtype != param_dtype:
            return value.to(param_dtype)
        return value

    def root_pre_forward(module, args, kwargs):
        root.pre_forward()
        if not calls_block_hooks:
            # this model's forward does not announce its blocks: every unit must be whole now
            for u in units:
                u.pre_forward()
        if param_dtype == torch.float32:
            return None
        # floating-point inputs (images, diffusion times, soft tokens) enter in the parameter dtype
        return tuple(_to_param_dtype(a) for a in args), {k: _to_param_dtype(v) for k, v in kwargs.items()}

    model.register_forward_pre_hook(root_pre_forward, with_kwargs=True)
    # state_dict() hands out views of the flat buffers: they must be whole and current first
    model.register_state_dict_pre_hook(lambda module, prefix, keep_vars: state.wait_parameters())
    if reshard_after_forward and shard_group is not None and calls_block_hooks:
        # block units follow the memory-lean schedule; the root (embedding) and head units are used
        # at both ends of every pass and stay whole, as the reference's outermost wrapper does
        for u in block_units.values():
            if u is not head_unit:
                u.enable_reshard()
        fused_all_gather = fused_reduce_scatter = False
    elif reshard_after_forward and shard_group is not None:
        from halite_b200.logging import logger

        logger.warning("reshard_after_forward: this model's forward does not announce its blocks, so its "
                       "parameters stay gathered")
    if fused_all_gather is None:
        import os

        fused_all_gather = os.environ.get("HB_FSDP_FUSED_GATHER", "0") == "1"
    if fused_all_gather and shard_group is not None and device.type == "cuda" and calls_block_hooks:
        enable_fused_gather(state)
    if fused_reduce_scatter is None:
        import os

        fused_reduce_scatter = os.environ.get("HB_FSDP_FUSED_REDUCE", "0") == "1"
    if fused_reduce_scatter and shard_group is not None and device.type == "cuda" and calls_block_hooks:
        enable_fused_reduce(state)
    return model


def apply_ddp(model, mesh=None, **kwargs):
    """Replicated data parallelism: same flat-buffer machinery with a shard group of one rank
    and gradient all-reduce over the replicate dimension."""
    return apply_fsdp(model, mesh, **kwargs)
