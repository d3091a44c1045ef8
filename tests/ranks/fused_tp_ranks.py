"""Rank script (one process per GPU, NCCL): fused all-gather->GEMM and GEMM->reduce-scatter over
symmetric memory against the NCCL + GEMM pairs they replace, with device-side timing (max over
ranks). Launch: torchrun --nproc-per-node N tests/ranks/fused_tp_ranks.py [--time]"""

import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from halite_b200 import ops  # noqa: E402
from halite_b200.ops import gemm  # noqa: E402
from halite_b200.parallel.fused_tp import FusedAllGatherGemm, FusedGemmReduceScatter  # noqa: E402
from halite_b200.parallel.symm import SymmetricHeap  # noqa: E402


def timed(fn, n=10, warm=3):
    for _ in range(warm):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / n], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("cpu:gloo,cuda:nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    group = dist.group.WORLD
    do_time = "--time" in sys.argv
    big = "--big" in sys.argv
    rows, K, N = (16384 // world, 4096, 6144 // world * 2) if big else (1024, 1024, 1536)
    N = N // 256 * 256
    heap = SymmetricHeap(rows * world * max(K, N) * 2 * 6 + (1 << 20), group)
    if rank == 0:
        print("heap backend", heap.backend, "multicast", hex(heap.multicast_ptr), flush=True)
    torch.manual_seed(1234 + rank)
    result = {"world": world, "rows_per_rank": rows, "K": K, "N": N, "backend": heap.backend}

    # ---------------- all-gather -> GEMM
    ag = FusedAllGatherGemm(heap, rows, K)
    w_col = (0.05 * torch.randn(N, K, device="cuda")).bfloat16()
    worst = 0.0
    for it in range(4):
        x = torch.randn(rows, K, device="cuda").bfloat16()
        y = ag(w_col, x_shard=x)
        full = torch.empty(world * rows, K, device="cuda", dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, x)
        ref = full.float() @ w_col.float().t()
        worst = max(worst, ((y.float() - ref).abs().max() / ref.abs().max()).item())
    torch.cuda.synchronize()
    ops.check_status()
    result["ag_gemm_rel_err"] = worst
    assert worst < 6e-3, worst

    # ---------------- GEMM -> reduce-scatter
    rs = FusedGemmReduceScatter(heap, rows, N)
    w_row = (0.05 * torch.randn(N, K, device="cuda")).bfloat16()
    worst = 0.0
    for it in range(4):
        x = torch.randn(world * rows, K, device="cuda").bfloat16()
        out = rs(x, w_row)
        part = (x.float() @ w_row.float().t())
        ref = torch.empty(rows, N, device="cuda")
        dist.reduce_scatter_tensor(ref, part)
        worst = max(worst, ((out.float() - ref).abs().max() / ref.abs().max()).item())
        dist.barrier()
    torch.cuda.synchronize()
    ops.check_status()
    result["gemm_rs_rel_err"] = worst
    assert worst < 2e-2, worst

    if do_time:
        x = torch.randn(rows, K, device="cuda").bfloat16()
        full = torch.empty(world * rows, K, device="cuda", dtype=torch.bfloat16)
        ybuf = torch.empty(world * rows, N, device="cuda", dtype=torch.bfloat16)

        def fused_ag():
            ag(w_col, out=ybuf, x_shard=x)

        def nccl_ag():
            dist.all_gather_into_tensor(full, x)
            gemm(full, w_col, out=ybuf)

        def gemm_only():
            gemm(full, w_col, out=ybuf)

        xs = torch.randn(world * rows, K, device="cuda").bfloat16()
        part = torch.empty(world * rows, N, device="cuda", dtype=torch.bfloat16)
        red = torch.empty(rows, N, device="cuda", dtype=torch.bfloat16)

        def fused_rs():
            rs(xs, w_row, out=red)

        def nccl_rs():
            gemm(xs, w_row, out=part)
            dist.reduce_scatter_tensor(red, part)

        result["t_fused_ag_gemm_ms"] = timed(fused_ag)
        result["t_nccl_ag_then_gemm_ms"] = timed(nccl_ag)
        result["t_gemm_only_ms"] = timed(gemm_only)
        result["t_fused_gemm_rs_ms"] = timed(fused_rs)
        result["t_gemm_then_nccl_rs_ms"] = timed(nccl_rs)
        flops = 2.0 * world * rows * K * N
        link = 770e9
        ag_bytes = (world - 1) * rows * K * 2
        rs_bytes = (world - 1) * rows * N * 2
        peak = 1.39e15
        result["ag_gemm_roofline_ms"] = max(flops / peak, ag_bytes / link) * 1e3
        result["gemm_rs_roofline_ms"] = max(flops / peak, rs_bytes / link) * 1e3
        ops.check_status()
    if rank == 0:
        print("RESULT " + json.dumps(result), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
