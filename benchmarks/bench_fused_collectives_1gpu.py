"""The four fused compute + collective GEMM modes on ONE GPU, at training sizes:

    python -m benchmarks.bench_fused_collectives_1gpu [--mode all|ag_gemm|gemm_rs|fsdp_gather|fsdp_reduce] [--iters 5]

The peers' buffers are stand-in tensors in this GPU's memory and their flags are pre-set, so the
copy CTAs, the flag-gated tiles, the scatter epilogue and the in-kernel reduction all run inside a
single launch (kernels that wait on one another must never run as separate launches on one GPU).
What this measures is therefore the kernels' own cost with local-memory "peers": the time a mode
adds to the plain GEMM of the same shape when the link is not the limit. The two-GPU numbers are
in `tests/ranks/fused_tp_ranks.py` / `profiles/fused_tp_collective_gemm_2gpu.md`. It is also the
small, single-GPU program the ncu captures of these kernels run.

Timed with CUDA events around one launch, 3 warm-up launches, a 256 MB buffer rewritten between
launches. Prints one JSON line per mode.
"""

from __future__ import annotations

import argparse
import json

import torch


def _i32(n, val=0):
    return torch.full((n,), val, dtype=torch.int32, device="cuda")


def _timed(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.add_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def ag_gemm(iters, flush, world=2, rows=8192, K=4096, N=6144):
    """Tensor-parallel all-gather -> GEMM: tiles wait for the 128-row granules the copy CTAs bring in."""
    from halite_b200.ops import gemm

    rank = 0
    shards = [torch.randn(rows, K, device="cuda").bfloat16() for _ in range(world)]
    w = (0.05 * torch.randn(N, K, device="cuda")).bfloat16()
    staging = torch.zeros(world * rows, K, device="cuda", dtype=torch.bfloat16)
    staging[rank * rows:(rank + 1) * rows] = shards[rank]
    state = {"epoch": 0}
    ready, done = _i32(world, 1 << 30), _i32(world)
    flags, counter = _i32(world * rows // 128), _i32(1)

    def fused():
        state["epoch"] += 1
        gather = dict(
            src_ptrs=[0 if c == rank else shards[c].data_ptr() for c in range(world)],
            peer_done_ptrs=[0 if c == rank else done[c:].data_ptr() for c in range(world)],
            dst_ptr=staging.data_ptr(), chunk_bytes=rows * K * 2, granule_bytes=128 * K * 2, n_copy_ctas=16,
            flags_ptr=flags.data_ptr(), ready_ptr=ready.data_ptr(), done_counter_ptr=counter.data_ptr(),
            epoch=state["epoch"], dep=1, dep_row_bytes=K * 2, dep_base_offset=0, m_rot=rank * rows // 128,
            first_chunk=rank)
        return gemm(staging, w, gather=gather)

    full = torch.cat(shards, 0)
    t_fused = _timed(fused, iters, flush)
    t_plain = _timed(lambda: gemm(full, w), iters, flush)
    copied = (world - 1) * rows * K * 2
    return {"mode": "ag_gemm", "shape": [world * rows, N, K], "fused_ms": t_fused, "plain_gemm_ms": t_plain,
            "bytes_copied": copied, "tflops_fused": 2 * world * rows * N * K / t_fused / 1e9}


def gemm_rs(iters, flush, world=2, rows=8192, K=2048, N=4096):
    """GEMM -> reduce-scatter: the epilogue pushes the peers' row blocks, the last CTA adds what arrived."""
    from halite_b200.ops import gemm

    rank = 0
    x = torch.randn(world * rows, K, device="cuda").bfloat16()
    w = (0.05 * torch.randn(N, K, device="cuda")).bfloat16()
    partial = torch.zeros(rows, N, device="cuda", dtype=torch.bfloat16)
    peer_mem = torch.zeros(rows, N, device="cuda", dtype=torch.bfloat16)
    from_peer = torch.randn(rows, N, device="cuda").bfloat16()
    out = torch.zeros(rows, N, device="cuda", dtype=torch.bfloat16)
    my_flags, peer_flags, counter = _i32(world, 1 << 30), _i32(world), _i32(1)
    state = {"epoch": 0}

    def fused():
        state["epoch"] += 1
        scatter = dict(
            dst_ptrs=[partial.data_ptr() if c == rank else peer_mem.data_ptr() for c in range(world)],
            recv_ptrs=[0 if p == rank else from_peer.data_ptr() for p in range(world)],
            peer_flag_ptrs=[0 if c == rank else peer_flags[c:].data_ptr() for c in range(world)],
            my_flags_ptr=my_flags.data_ptr(), out_ptr=out.data_ptr(), cta_counter_ptr=counter.data_ptr(),
            rows_per_chunk=rows, rank=rank, epoch=state["epoch"])
        return gemm(x, w, out=partial, scatter=scatter)

    full_out = torch.empty(world * rows, N, device="cuda", dtype=torch.bfloat16)
    t_fused = _timed(fused, iters, flush)
    t_plain = _timed(lambda: gemm(x, w, out=full_out), iters, flush)
    return {"mode": "gemm_rs", "shape": [world * rows, N, K], "fused_ms": t_fused, "plain_gemm_ms": t_plain,
            "bytes_pushed": (world - 1) * rows * N * 2, "tflops_fused": 2 * world * rows * N * K / t_fused / 1e9}


def _carrier():
    # the GEMM that carries the job: a down-projection forward of the 3B model (32768 tokens)
    M, N, K = 32768, 3072, 8192
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (0.02 * torch.randn(N, K, device="cuda")).bfloat16()
    return x, w, (M, N, K)


def fsdp_gather(iters, flush, world=8, unit_numel=100_663_296):
    """FSDP parameter gather carried by a GEMM launch: 16 CTAs copy the peers' bf16 shards into the
    unit's flat buffer while the other CTAs compute (no tile waits for the copy)."""
    from halite_b200.ops import gemm

    rank = 0
    chunk = unit_numel // world
    shards = [torch.randn(chunk, device="cuda").bfloat16() for _ in range(world)]
    flat = torch.zeros(unit_numel, device="cuda", dtype=torch.bfloat16)
    ready, done, counter = _i32(world, 1 << 30), _i32(world), _i32(1)
    gran = 256 * 1024
    flags = _i32(world * ((chunk * 2 + gran - 1) // gran))
    x, w, shape = _carrier()
    state = {"epoch": 0}

    def fused():
        state["epoch"] += 1
        gather = dict(
            src_ptrs=[0 if c == rank else shards[c].data_ptr() for c in range(world)],
            peer_done_ptrs=[0 if c == rank else done[c:].data_ptr() for c in range(world)],
            dst_ptr=flat.data_ptr(), chunk_bytes=chunk * 2, granule_bytes=gran, n_copy_ctas=16,
            flags_ptr=flags.data_ptr(), ready_ptr=ready.data_ptr(), done_counter_ptr=counter.data_ptr(),
            epoch=state["epoch"], dep=0, dep_row_bytes=0, dep_base_offset=0, first_chunk=rank)
        return gemm(x, w, gather=gather)

    t_fused = _timed(fused, iters, flush)
    t_plain = _timed(lambda: gemm(x, w), iters, flush)
    return {"mode": "fsdp_gather", "carrier_shape": list(shape), "fused_ms": t_fused, "plain_gemm_ms": t_plain,
            "bytes_copied": (world - 1) * chunk * 2}


def fsdp_reduce(iters, flush, world=8, unit_numel=100_663_296):
    """FSDP gradient reduction carried by a GEMM launch: 32 CTAs read this rank's range of every
    rank's fp32 gradient buffer, add in rank order, scale and write the shard."""
    from halite_b200.ops import gemm

    rank = 0
    n = unit_numel // world
    grads = [torch.randn(n, device="cuda") for _ in range(world)]     # this rank's range of each rank's buffer
    out = torch.zeros(n, device="cuda")
    ready, done, counter = _i32(world, 1 << 30), _i32(world), _i32(1)
    x, w, shape = _carrier()
    state = {"epoch": 0}

    def fused():
        state["epoch"] += 1
        gather = dict(
            src_ptrs=[g.data_ptr() for g in grads], dst_ptr=0, chunk_bytes=16, granule_bytes=16,
            n_copy_ctas=32, flags_ptr=0, ready_ptr=ready.data_ptr(), done_counter_ptr=counter.data_ptr(),
            peer_done_ptrs=[0 if c == rank else done[c:].data_ptr() for c in range(world)],
            epoch=state["epoch"], dep=0, dep_row_bytes=0, first_chunk=rank,
            reduce_out_ptr=out.data_ptr(), reduce_numel=n, reduce_scale=1.0 / world)
        return gemm(x, w, gather=gather)

    t_fused = _timed(fused, iters, flush)
    t_plain = _timed(lambda: gemm(x, w), iters, flush)
    return {"mode": "fsdp_reduce", "carrier_shape": list(shape), "fused_ms": t_fused, "plain_gemm_ms": t_plain,
            "bytes_read": world * n * 4, "bytes_written": n * 4}


MODES = {"ag_gemm": ag_gemm, "gemm_rs": gemm_rs, "fsdp_gather": fsdp_gather, "fsdp_reduce": fsdp_reduce}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="all", choices=["all", *MODES])
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args(argv)

    from halite_b200 import ops

    torch.manual_seed(0)
    flush = torch.zeros(64 * 1024 * 1024, device="cuda")
    out = []
    for name, fn in MODES.items():
        if args.mode in ("all", name):
            row = fn(args.iters, flush)
            torch.cuda.synchronize()
            ops.check_status()
            print(json.dumps(row), flush=True)
            out.append(row)
    return out


if __name__ == "__main__":
    main()
