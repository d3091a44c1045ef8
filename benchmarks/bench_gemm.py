"""Micro-benchmark of the tcgen05 GEMM against cuBLAS (torch.matmul) on the shapes of a
transformer step: `python -m benchmarks.bench_gemm [--tokens 32768] [--dim 3072] ...`.

Each case is timed with CUDA events over `--iters` launches after warm-up, with a buffer larger
than L2 rewritten between launches so operands start cold. Prints one JSON line per case.
"""

from __future__ import annotations

import argparse
import json

import torch

from halite_b200 import ops
from halite_b200.ops.linear import gemm


def _time(fn, iters, flush):
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--dim", type=int, default=3072)
    ap.add_argument("--qkv", type=int, default=5120)
    ap.add_argument("--ff", type=int, default=8192)
    ap.add_argument("--vocab", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--layers", default="", help="comma list of layer names to run (default: all)")
    ap.add_argument("--cases", default="", help="comma list among fwd,dgrad,wgrad_f32 (default: all)")
    ap.add_argument("--no-cublas", action="store_true", help="time only this package's kernel")
    ap.add_argument("--decode", type=int, default=0, metavar="BATCH",
                    help="time the forward GEMMs at this many rows (a decode step) instead of the training shapes")
    ap.add_argument("--compare-schedules", action="store_true",
                    help="time the CTA-pair kernel with dynamic and with fixed work shares, back to back")
    ap.add_argument("--block-n", default="0",
                    help="comma list of tiles to time: 64 / 128 / 256 (one CTA per tile), 512 (CTA pair, 256 x 256), "
                         "0 = the launcher's choice")
    args = ap.parse_args()
    dev = "cuda"
    flush = torch.zeros(192 << 20, dtype=torch.uint8, device=dev)       # > 126 MB of L2
    T = args.decode or args.tokens
    block_ns = [int(b) for b in args.block_n.split(",")]
    layers = [("qkv", args.dim, args.qkv), ("attn_out", args.dim, args.dim), ("up_gate", args.dim, 2 * args.ff),
              ("down", args.ff, args.dim)]
    if args.vocab:
        layers.append(("head", args.dim, args.vocab))
    want_layers = set(filter(None, args.layers.split(",")))
    want_cases = set(filter(None, args.cases.split(",")))
    for name, k, n in layers:
        if want_layers and name not in want_layers:
            continue
        x = torch.randn(T, k, device=dev).bfloat16()
        w = (0.02 * torch.randn(n, k, device=dev)).bfloat16()
        dy = torch.randn(T, n, device=dev).bfloat16()
        y = torch.empty(T, n, device=dev, dtype=torch.bfloat16)
        dx = torch.empty(T, k, device=dev, dtype=torch.bfloat16)
        dw = torch.empty(n, k, device=dev, dtype=torch.float32)
        dwb = torch.empty(n, k, device=dev, dtype=torch.bfloat16)
        def cases_for(bn):
            return {
                "fwd": lambda: gemm(x, w, out=y, block_n=bn),
                "dgrad": lambda: gemm(dy, w, out=dx, b_mn=True, block_n=bn),
                "wgrad_f32": lambda: gemm(dy, x, out=dw, a_mn=True, b_mn=True, block_n=bn),
            }

        lib_cases = {
            "fwd": lambda: torch.matmul(x, w.t(), out=y),
            "dgrad": lambda: torch.matmul(dy, w, out=dx),
            "wgrad_f32": lambda: torch.matmul(dy.t(), x, out=dwb),
        }
        flops = 2.0 * T * k * n
        for case, lib in lib_cases.items():
            if (want_cases and case not in want_cases) or (args.decode and case != "fwd"):
                continue
            t_lib = float("nan") if args.no_cublas else _time(lib, args.iters, flush)
            variants = [(bn, None) for bn in block_ns]
            if args.compare_schedules:
                variants = [(512, True), (512, False)]
            for bn, dyn in variants:
                if dyn is not None:
                    ops.ext().gemm_set_dynamic_schedule(dyn, True)
                t_ours = _time(cases_for(bn)[case], args.iters, flush)
                print(json.dumps({"layer": name, "case": case, "M_N_K": [T, n, k] if case == "fwd" else None,
                                  "block_n": bn, "dynamic": dyn, "ours_ms": round(t_ours, 4), "cublas_ms": round(t_lib, 4),
                                  "ours_tflops": round(flops / t_ours / 1e9, 1),
                                  "cublas_tflops": round(flops / t_lib / 1e9, 1),
                                  "ratio": round(t_lib / t_ours, 3)}), flush=True)


if __name__ == "__main__":
    main()
