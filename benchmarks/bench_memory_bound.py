"""Achieved memory bandwidth of the memory-bound training kernels at transformer-step sizes:

    python -m benchmarks.bench_memory_bound [--tokens 32768] [--dim 3072] [--ff 8192]

Each op is timed with CUDA events over `--iters` launches after warm-up, a buffer larger than L2
rewritten between launches; bytes are the op's algorithmic traffic (every operand read once,
every result written once). Prints one JSON line per op with GB/s and, when the measured-peaks
file of the repository root is present, the fraction of the measured copy bandwidth.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from halite_b200 import ops
from halite_b200.ops.activation import gated_act
from halite_b200.ops.rope import rope_tables


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


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--dim", type=int, default=3072)
    ap.add_argument("--ff", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--ema-seqs", type=int, default=16, help="sequences in the packed row of the EMA cases")
    ap.add_argument("--ema-len", type=int, default=1024, help="chunk vectors per sequence in the EMA cases")
    ap.add_argument("--ema-dim", type=int, default=1536)
    args = ap.parse_args(argv)
    dev = "cuda"
    C = ops.ext()
    flush = torch.zeros(192 << 20, dtype=torch.uint8, device=dev)
    peak = None
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            peak = float(json.load(f)["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        pass
    T, D, FF = args.tokens, args.dim, args.ff
    bf = torch.bfloat16
    x, r, g = (torch.randn(T, D, device=dev, dtype=bf) for _ in range(3))
    w = torch.ones(D, device=dev, dtype=bf)
    act_bytes = T * D * 2
    cases = []

    def norm_fwd(res):
        return lambda: C.rmsnorm_fwd(x, res, w, 1e-5, 0.0, res is not None)

    cases.append(("rmsnorm_fwd", norm_fwd(None), 2 * act_bytes))
    cases.append(("rmsnorm_fwd_residual", norm_fwd(r), 4 * act_bytes))
    y, h, rstd = C.rmsnorm_fwd(x, r, w, 1e-5, 0.0, True)
    cases.append(("rmsnorm_bwd", lambda: C.rmsnorm_bwd(g, h, w, rstd, None, 0.0), 5 * act_bytes))
    cases.append(("rmsnorm_bwd_dres", lambda: C.rmsnorm_bwd(g, h, w, rstd, r, 0.0), 6 * act_bytes))

    H, Hk, Dh = args.heads, args.kv_heads, args.head_dim
    qkv = torch.randn(1, T, (H + 2 * Hk) * Dh, device=dev, dtype=bf)
    inv = 1.0 / (500000 ** (torch.arange(0, Dh, 2).float() / Dh))
    cos, sin = rope_tables(inv, 8192, dev)
    pos = (torch.arange(T, device=dev) % 4096).contiguous()
    qk = qkv[..., : (H + Hk) * Dh].unflatten(-1, (H + Hk, Dh))
    cases.append(("rope_qk_in_place", lambda: C.rope_(qk, cos, sin, pos, Dh, True, False), 2 * T * (H + Hk) * Dh * 2))
    dq = torch.randn(1, T, H, Dh, device=dev, dtype=bf)
    gq = qkv[..., : H * Dh].unflatten(-1, (H, Dh))
    cases.append(("rope_rotate_into_packed_grad", lambda: C.rope_copy(dq, gq, cos, sin, pos, Dh, True, True),
                  2 * T * H * Dh * 2))

    gate, up, dout = (torch.randn(T, FF, device=dev, dtype=bf) for _ in range(3))
    cases.append(("swiglu_fwd", lambda: gated_act(gate, up, "silu"), 3 * T * FF * 2))
    cases.append(("swiglu_bwd", lambda: C.gated_act_bwd(gate, up, dout, 0, None, None), 5 * T * FF * 2))

    # the H-Net dechunk EMA: the recurrence kernel and, for its time only, the chunked formulation
    from halite_b200.models.models.mamba2 import ssd_scan
    from halite_b200.ops.scan import linear_scan

    S, L, De = args.ema_seqs, args.ema_len, args.ema_dim
    ex = torch.randn(S * L, De, device=dev, dtype=bf)
    ep = torch.rand(S * L, device=dev).clamp(0.05, 0.95)
    eq, one = 1 - ep, torch.ones_like(ep)
    eg = torch.randn(S * L, De, device=dev)
    cu = torch.arange(0, S * L + 1, L, device=dev, dtype=torch.int32)
    seq_idx = torch.arange(S, device=dev, dtype=torch.int32).repeat_interleave(L)[None]
    cases.append(("ema_scan_fwd", lambda: linear_scan(ex, eq, ep, cu), S * L * De * 6))
    cases.append(("ema_scan_adjoint", lambda: linear_scan(eg, eq, one, cu, reverse=True), S * L * De * 8))

    def chunked():
        dt = torch.log(1 / eq)[None]
        xs = (ex.float()[None] / dt[..., None]).view(1, S * L, 1, De)
        return ssd_scan(xs, dt[..., None], -torch.ones(1, device=dev), ep.view(1, -1, 1, 1),
                        torch.ones(1, S * L, 1, 1, device=dev), chunk_size=64, seq_idx=seq_idx)[0]

    cases.append(("ema_chunked_formulation_fwd", chunked, S * L * De * 6))

    for name, fn, nbytes in cases:
        ms = _time(fn, args.iters, flush)
        gbs = nbytes / ms / 1e6
        out = {"op": name, "ms": round(ms, 4), "bytes": nbytes, "gb_per_s": round(gbs, 1)}
        if peak:
            out["of_measured_copy_bandwidth"] = round(gbs / peak, 3)
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
