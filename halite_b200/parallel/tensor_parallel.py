"""Tensor parallelism with sequence-parallel activations (reference: transformers/parallelize.py
:130-142,164-185 and the per-module plans in transformers/attention.py:249-259,359-371,
transformers/feedforward.py:106-225, transformers/embedding.py:46-51).

Between blocks every TP rank holds a contiguous 1/tp slice of the flattened tokens
(`[tokens / tp, dim]`); norms and residual adds run on that slice. Entering attention or the
feed-forward the slices are all-gathered and the column-parallel projections follow; leaving,
the row-parallel projection's partial sums are reduce-scattered back to token slices.

On CUDA both pairs are ONE kernel each (`FusedAllGatherGemm`, `FusedGemmReduceScatter`); on CPU
(Gloo) the same autograd functions fall back to collectives + `F.linear`, which is what the
multi-process CPU tests run.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

import halite_b200.ops as ops
from halite_b200.ops.linear import gemm


class TPContext:
    """Per-model tensor-parallel state: group, rank, symmetric heap and fused operator cache."""

    def __init__(self, group, heap_bytes=None, device=None, fused=None):
        self.group = group
        self.size = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.device = device
        self.batch_shape = None        # (batch, seq) of the current forward, set by the decoder
        self.heap = None
        self.heap_bytes = heap_bytes
        self._ag = {}
        self._rs = {}
        self.fused = fused

    def use_fused(self, x):
        if self.size == 1 or not ops.use_sm100(x):
            return False
        if self.fused is None:
            self.fused = True
        return self.fused

    def _ensure_heap(self, device):
        if self.heap is None:
            from halite_b200.parallel.symm import SymmetricHeap

            self.heap = SymmetricHeap(self.heap_bytes or (2 << 30), self.group, device)
        return self.heap

    def ag_op(self, rows, k, device):
        key = (rows, k)
        if key not in self._ag:
            from halite_b200.parallel.fused_tp import FusedAllGatherGemm

            self._ag[key] = FusedAllGatherGemm(self._ensure_heap(device), rows, k)
        return self._ag[key]

    def rs_op(self, rows, n, device):
        key = (rows, n)
        if key not in self._rs:
            from halite_b200.parallel.fused_tp import FusedGemmReduceScatter

            self._rs[key] = FusedGemmReduceScatter(self._ensure_heap(device), rows, n)
        return self._rs[key]


# --------------------------------------------------------------------------- plain collectives

def _all_gather_rows(x, ctx):
    out = x.new_empty(ctx.size * x.shape[0], *x.shape[1:])
    dist.all_gather_into_tensor(out, x.contiguous(), group=ctx.group)
    return out


def _reduce_scatter_rows(x, ctx):
    rows = x.shape[0] // ctx.size
    if dist.get_backend(ctx.group) == "gloo":
        x = x.contiguous().clone()
        dist.all_reduce(x, group=ctx.group)
        return x[ctx.rank * rows:(ctx.rank + 1) * rows].clone()
    out = x.new_empty(rows, *x.shape[1:])
    dist.reduce_scatter_tensor(out, x.contiguous(), group=ctx.group)
    return out


class _GatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _all_gather_rows(x, tp)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_rows(g, ctx.tp), None


class _ScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _reduce_scatter_rows(x, tp)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_rows(g, ctx.tp), None


class _CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward (input replicated over TP, used by sharded weights)."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.tp.group)
        return g, None


class _GatherCols(torch.autograd.Function):
    """[T, n] column shards -> [T, tp * n]; backward keeps this rank's columns."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp, ctx.n = tp, x.shape[-1]
        full = _all_gather_rows(x.contiguous(), tp)                  # [tp * T, n]
        return full.view(tp.size, x.shape[0], -1).permute(1, 0, 2).reshape(x.shape[0], -1)

    @staticmethod
    def backward(ctx, g):
        return g[:, ctx.tp.rank * ctx.n:(ctx.tp.rank + 1) * ctx.n].contiguous(), None


def gather_cols(x, tp):
    return x if tp.size == 1 else _GatherCols.apply(x, tp)


def gather_rows(x, tp):
    return x if tp.size == 1 else _GatherRows.apply(x, tp)


def scatter_rows(x, tp):
    return x if tp.size == 1 else _ScatterRows.apply(x, tp)


# --------------------------------------------------------------------------- fused layers

def _wgrad(dy, x, weight):
    """dW = dy^T x into the flat gradient buffer when the weight has one."""
    main = getattr(weight, "_hb_grad", None)
    if ops.use_sm100(dy):
        if main is not None:
            owner = getattr(weight, "_hb_grad_owner", None)
            acc = owner.mark_written(weight) if owner is not None else False
            gemm(dy, x, out=main, a_mn=True, b_mn=True, accumulate=acc)
            return None
        return gemm(dy, x, a_mn=True, b_mn=True, out_dtype=weight.dtype)
    dw = dy.t().to(weight.dtype) @ x.to(weight.dtype)
    if main is not None:
        # same main-grad protocol on the PyTorch path (fused views are not autograd leaves
        # that anything reads)
        owner = getattr(weight, "_hb_grad_owner", None)
        acc = owner.mark_written(weight) if owner is not None else False
        if acc:
            main.add_(dw)
        else:
            main.copy_(dw)
        return None
    return dw


class _AGLinear(torch.autograd.Function):
    """y = all_gather(x_local) @ W^T, W this rank's column shard [N/tp, K]."""

    @staticmethod
    def forward(ctx, x_local, weight, tp, keep_gathered):
        ctx.tp = tp
        ctx.weight_ref = weight
        x2 = x_local.reshape(-1, x_local.shape[-1])
        fused = tp.use_fused(x2) and x2.shape[0] % 128 == 0
        if fused:
            op = tp.ag_op(x2.shape[0], x2.shape[1], x2.device)
            y = op(weight, x_shard=x2)
            x_full = op.staging((op.call - 1) % op.n_buf)
            if keep_gathered:
                x_full = x_full.clone()
        else:
            x_full = _all_gather_rows(x2, tp)
            y = ops.linear(x_full, weight) if ops.use_sm100(x_full) else F.linear(x_full, weight)
        ctx.save_for_backward(x2, weight)
        ctx.fused = fused
        if keep_gathered:
            ctx.mark_non_differentiable(x_full)
            return y, x_full
        return y, None

    @staticmethod
    def backward(ctx, dy, _unused=None):
        x2, weight = ctx.saved_tensors
        tp = ctx.tp
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        x_full = _all_gather_rows(x2, tp)          # re-gather instead of keeping the activation
        dw = _wgrad(dy2, x_full, ctx.weight_ref)
        if ctx.fused and dy2.shape[0] % (128 * tp.size) == 0:
            rs = tp.rs_op(x2.shape[0], weight.shape[1], dy2.device)
            dx = rs(dy2, weight, b_mn=True)
        else:
            dx_full = gemm(dy2, weight, b_mn=True) if ops.use_sm100(dy2) else dy2 @ weight
            dx = _reduce_scatter_rows(dx_full, tp)
        return dx.view(x2.shape), dw, None, None


class _LinearRS(torch.autograd.Function):
    """out_local = reduce_scatter(x @ W^T), W this rank's row shard [N, K/tp]."""

    @staticmethod
    def forward(ctx, x, weight, tp):
        ctx.tp = tp
        ctx.weight_ref = weight
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0] // tp.size
        fused = tp.use_fused(x2) and rows % 128 == 0 and x2.shape[0] % tp.size == 0
        if fused:
            out = tp.rs_op(rows, weight.shape[0], x2.device)(x2, weight)
        else:
            y = ops.linear(x2, weight) if ops.use_sm100(x2) else F.linear(x2, weight)
            out = _reduce_scatter_rows(y, tp)
        ctx.save_for_backward(x2, weight)
        ctx.fused = fused
        return out

    @staticmethod
    def backward(ctx, dout):
        x2, weight = ctx.saved_tensors
        tp = ctx.tp
        d2 = dout.reshape(-1, dout.shape[-1]).contiguous()
        if ctx.fused:
            op = tp.ag_op(d2.shape[0], d2.shape[1], d2.device)
            dx = op(weight, x_shard=d2, b_mn=True)       # all_gather(dout) @ W, one kernel
            dy_full = op.staging((op.call - 1) % op.n_buf)
        else:
            dy_full = _all_gather_rows(d2, tp)
            dx = gemm(dy_full, weight, b_mn=True) if ops.use_sm100(dy_full) else dy_full @ weight
        dw = _wgrad(dy_full, x2, ctx.weight_ref)
        return dx.view(x2.shape), dw, None


def ag_linear(x_local, weight, tp, keep_gathered=False):
    """Column-parallel linear on token-sharded input. Returns (y, gathered input or None)."""
    if tp.size == 1:
        return ops.linear(x_local, weight), (x_local if keep_gathered else None)
    return _AGLinear.apply(x_local, weight, tp, keep_gathered)


def linear_rs(x, weight, tp):
    """Row-parallel linear whose summed output is scattered back to token shards."""
    if tp.size == 1:
        return ops.linear(x, weight)
    return _LinearRS.apply(x, weight, tp)


# --------------------------------------------------------------------------- embedding / loss

class _VocabParallelEmbedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, tp):
        v = weight.shape[0]
        lo = tp.rank * v
        local = ids - lo
        own = (local >= 0) & (local < v)
        out = F.embedding(local.clamp(0, v - 1), weight)
        out = out * own.unsqueeze(-1).to(out.dtype)
        ctx.save_for_backward(local, own)
        ctx.tp, ctx.v = tp, v
        ctx.weight_ref = weight
        return _reduce_scatter_rows(out.reshape(-1, out.shape[-1]), tp)

    @staticmethod
    def backward(ctx, g):
        local, own = ctx.saved_tensors
        g_full = _all_gather_rows(g.contiguous(), ctx.tp)
        w = ctx.weight_ref
        grad = torch.zeros(ctx.v, g_full.shape[-1], dtype=g_full.dtype, device=g_full.device)
        rows = local.reshape(-1)[own.reshape(-1)]
        grad.index_add_(0, rows, g_full[own.reshape(-1)])
        return None, grad.to(w.dtype), None


def vocab_parallel_embedding(ids, weight, tp):
    """ids [B, S] (same on every TP rank), weight [V/tp, D] -> token shard [B*S/tp, D]."""
    return _VocabParallelEmbedding.apply(ids, weight, tp)


class _VocabParallelCE(torch.autograd.Function):
    """Cross entropy over a vocabulary split across TP ranks, without gathering logits: each rank
    reduces its shard to (log-sum-exp, target logit), the pairs are combined across ranks, and the
    gradient uses the global log-sum-exp. hidden: [T, D] (gathered), weight: [V/tp, D]."""

    @staticmethod
    def forward(ctx, hidden, weight, target, tp, ignore_index, chunk_rows):
        T, V = hidden.shape[0], weight.shape[0]
        lo = tp.rank * V
        losses = torch.empty(T, dtype=torch.float32, device=hidden.device)
        lses = torch.empty(T, dtype=torch.float32, device=hidden.device)
        chunk = chunk_rows or max(256, min(T, (1 << 30) // (V * 2)))
        on_gpu = ops.use_sm100(hidden)
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            if on_gpu:
                lg = gemm(hidden[s:e], weight)
                res = ops.ext().cross_entropy(lg, target[s:e].contiguous(), None, ignore_index, 0.0, 0.0,
                                              1.0, 0.0, 1.0, None, None, False, lo)
                lse_l, xt_l = res[1], res[1] - res[0]
                xt_l = torch.where(target[s:e] == ignore_index, torch.zeros_like(xt_l), xt_l)
            else:
                lg = F.linear(hidden[s:e], weight).float()
                lse_l = torch.logsumexp(lg, -1)
                loc = target[s:e] - lo
                own = (loc >= 0) & (loc < V)
                xt_l = torch.where(own, lg.gather(-1, loc.clamp(0, V - 1).unsqueeze(-1)).squeeze(-1),
                                   torch.zeros_like(lse_l))
            pair = torch.stack([lse_l, xt_l], 0).contiguous()
            gathered = pair.new_empty(tp.size, *pair.shape)
            dist.all_gather_into_tensor(gathered.view(-1), pair.view(-1), group=tp.group)
            lse = torch.logsumexp(gathered[:, 0], 0)
            xt = gathered[:, 1].sum(0)
            valid = target[s:e] != ignore_index
            losses[s:e] = torch.where(valid, lse - xt, torch.zeros_like(lse))
            lses[s:e] = lse
        ctx.save_for_backward(hidden, weight, target, lses)
        ctx.tp, ctx.ignore_index, ctx.chunk, ctx.lo = tp, ignore_index, chunk, lo
        ctx.weight_ref = weight
        return losses

    @staticmethod
    def backward(ctx, g):
        hidden, weight, target, lses = ctx.saved_tensors
        T, V = hidden.shape[0], weight.shape[0]
        tp, lo = ctx.tp, ctx.lo
        on_gpu = ops.use_sm100(hidden)
        g = g.reshape(-1).float().contiguous()
        dh = torch.empty_like(hidden)
        wref = ctx.weight_ref
        main = getattr(wref, "_hb_grad", None)
        acc = False
        if main is not None and on_gpu:
            owner = getattr(wref, "_hb_grad_owner", None)
            acc = owner.mark_written(wref) if owner is not None else False
            dw = main
        else:
            dw = torch.zeros(weight.shape, dtype=torch.float32, device=hidden.device)
        for s in range(0, T, ctx.chunk):
            e = min(T, s + ctx.chunk)
            if on_gpu:
                lg = gemm(hidden[s:e], weight)
                # d logit = g * (p - onehot): the log-prob backward kernel with upstream -g
                ops.ext().logprob_entropy_bwd_(lg, target[s:e].contiguous(), lses[s:e].contiguous(), None,
                                               (-g[s:e]).contiguous(), None, None, lg, ctx.ignore_index, 1.0, lo)
                gemm(lg, weight, out=dh[s:e], b_mn=True)
                gemm(lg, hidden[s:e], out=dw, a_mn=True, b_mn=True, accumulate=acc or s > 0)
            else:
                lg = F.linear(hidden[s:e], weight).float()
                p = (lg - lses[s:e].unsqueeze(-1)).exp()
                loc = target[s:e] - lo
                own = (loc >= 0) & (loc < V) & (target[s:e] != ctx.ignore_index)
                p[own, loc[own]] -= 1.0
                p = p * (g[s:e] * (target[s:e] != ctx.ignore_index)).unsqueeze(-1)
                dh[s:e] = (p @ weight.float()).to(dh.dtype)
                dw += p.t() @ hidden[s:e].float()
        # dh is this rank's partial sum over its vocabulary shard: the ranks' partials are added
        # by the backward of the gather that produced `hidden` (a reduce-scatter)
        gw = None if (main is not None and on_gpu) else dw.to(weight.dtype)
        return dh, gw, None, None, None, None


def vocab_parallel_cross_entropy(hidden, weight, target, tp, ignore_index=-100, chunk_rows=None):
    return _VocabParallelCE.apply(hidden, weight, target.reshape(-1), tp, ignore_index, chunk_rows)


# --------------------------------------------------------------------------- applying the plan

def _shard(param, dim, tp):
    n = param.shape[dim] // tp.size
    if param.shape[dim] % tp.size:
        raise ValueError(f"dimension {dim} of size {param.shape[dim]} is not divisible by tp={tp.size}")
    if param.is_meta:
        shape = list(param.shape)
        shape[dim] = n
        return nn.Parameter(torch.empty(shape, dtype=param.dtype, device="meta"), requires_grad=param.requires_grad)
    return nn.Parameter(param.detach().narrow(dim, tp.rank * n, n).clone(), requires_grad=param.requires_grad)


def _shard_linear(lin, how, tp, attn=None):
    if how in ("colwise", "colwise_gated", "colwise_qkv", "vocab_head"):
        if how == "colwise_gated":
            # rows are [gate | up]: shard each half so every rank keeps matching pairs
            w = lin.weight
            half = w.shape[0] // 2
            if w.is_meta:
                lin.weight = _shard(w, 0, tp)
            else:
                n = half // tp.size
                lin.weight = nn.Parameter(torch.cat([w.detach()[tp.rank * n:(tp.rank + 1) * n],
                                                     w.detach()[half + tp.rank * n: half + (tp.rank + 1) * n]], 0),
                                          requires_grad=w.requires_grad)
        elif how == "colwise_qkv" and attn is not None:
            w = lin.weight
            hq, hk, d = attn.n_heads * attn.head_dim, attn.kv_heads * attn.head_dim, attn.head_dim
            if w.is_meta:
                lin.weight = _shard(w, 0, tp)
            else:
                parts = []
                for start, size in ((0, hq), (hq, hk), (hq + hk, hk)):
                    n = size // tp.size
                    parts.append(w.detach()[start + tp.rank * n: start + (tp.rank + 1) * n])
                lin.weight = nn.Parameter(torch.cat(parts, 0), requires_grad=w.requires_grad)
        else:
            lin.weight = _shard(lin.weight, 0, tp)
        if getattr(lin, "bias", None) is not None:
            lin.bias = _shard(lin.bias, 0, tp)
        lin.out_features = lin.weight.shape[0]
    elif how == "rowwise":
        lin.weight = _shard(lin.weight, 1, tp)
        lin.in_features = lin.weight.shape[1]
    elif how == "vocab":
        lin.weight = _shard(lin.weight, 0, tp)
        lin.num_embeddings = lin.weight.shape[0]
    lin._hb_tp_kind = how


def _reserve_sms_for_other_groups(parallel_dims, tp):
    """The fused collective GEMMs spin on the tensor-parallel peer while they hold their SMs. When the
    ranks also run collectives of another group beside them (FSDP all-gathers and reduce-scatters over
    the data-parallel group), a peer can be held back by such a collective whose kernel finds no free SM
    on a third GPU that is itself spinning, and the ranks wait in a circle until the bounded waits give
    up. So the spinning launches leave `HB_TP_SM_MARGIN` SMs (default 20) free; the collective library
    must use no more CTAs than that (`NCCL_MAX_CTAS`, read by NCCL when its communicators are made)."""
    import os
    import warnings

    if tp.fused is False or not torch.cuda.is_available():
        return
    others = getattr(parallel_dims, "world_size", tp.size) // tp.size
    if others <= 1:
        return
    margin = int(os.environ.get("HB_TP_SM_MARGIN", "20"))
    ops.ext().gemm_set_peer_wait_sm_margin(margin)
    cap = os.environ.get("NCCL_MAX_CTAS")
    if cap is None or int(cap) > margin:
        warnings.warn(f"tensor parallelism with fused collective GEMMs beside data-parallel collectives: set "
                      f"NCCL_MAX_CTAS <= {margin} before the process groups are made (it is {cap}); otherwise the "
                      f"two can wait on each other until the kernels' bounded waits give up", stacklevel=3)


def apply_tp(model, parallel_dims, loss_parallel=True, enable_async_tp=True, heap_bytes=None, **unused):
    """Shard the model's linears / embedding / head over the `tp` mesh dimension according to
    each module's `tp_plan()` and switch the modules to their tensor-parallel forward."""
    group = parallel_dims.group("tp")
    tp = TPContext(group, heap_bytes=heap_bytes, fused=None if enable_async_tp else False)
    if tp.size == 1:
        return model
    for module in model.modules():
        plan_fn = getattr(module, "tp_plan", None)
        if plan_fn is None:
            continue
        attn = getattr(module, "attention", None)
        for name, how in plan_fn().items():
            sub = getattr(module, name, None)
            if sub is None or how == "sequence":
                continue
            _shard_linear(sub, how, tp, attn)
        module._hb_tp = tp
        if attn is not None:
            attn.n_heads //= tp.size
            if attn.n_key_value_heads is not None:
                attn.n_key_value_heads //= tp.size
            for a in ("n_heads", "n_key_value_heads"):
                if hasattr(module, a) and getattr(module, a) is not None:
                    setattr(module, a, getattr(module, a) // tp.size)
    model._hb_tp = tp
    model._hb_loss_parallel = loss_parallel
    _reserve_sms_for_other_groups(parallel_dims, tp)
    # parameters that stay replicated over TP but see only a token shard (norm scales) need
    # their gradients summed over the group
    sharded = set()
    for module in model.modules():
        if getattr(module, "_hb_tp_kind", None) is not None:
            sharded.update(id(p) for p in module.parameters(recurse=False))
    for p in model.parameters():
        if id(p) not in sharded:
            p._hb_tp_replicated = tp
    return model
