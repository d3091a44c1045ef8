"""Training attention, forward and backward: the repository's tcgen05 kernels against the
library kernels on the same box.

    python -m benchmarks.bench_attention [--batch 8] [--seq 4096] [--heads 24] [--kv-heads 8] [--dim 128]
                                         [--iters 10] [--packed 8192,4096,...] [--no-library]

Timed with CUDA events around `iters` launches after 3 warm-up launches; a 256 MB buffer is
rewritten between launches so that nothing is served from L2. FLOPs are 4 * S^2 * D per head and
sequence for the forward (halved when causal) and 2.5 x that for the backward.
"""

from __future__ import annotations

import argparse
import json

import torch


def timed(fn, iters, flush):
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
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--packed", default=None, help="comma-separated document lengths: one packed row instead of a batch")
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--no-library", action="store_true")
    ap.add_argument("--no-backward", action="store_true")
    args = ap.parse_args(argv)

    import torch.nn.functional as F

    from halite_b200 import ops
    from halite_b200.ops.attention import attention

    dev = torch.device("cuda")
    B, S, H, Hk, D = args.batch, args.seq, args.heads, args.kv_heads, args.dim
    cu = None
    if args.packed:
        lengths = [int(x) for x in args.packed.split(",")]
        B, S = 1, sum(lengths)
        bounds = [0]
        for n in lengths:
            bounds.append(bounds[-1] + n)
        cu = torch.tensor(bounds, device=dev, dtype=torch.int32)
        pairs = sum(n * n for n in lengths) / 2
    else:
        pairs = B * S * S / 2
        if args.window:
            pairs = B * S * min(args.window, S)
    flops_fwd = 4 * pairs * D * H
    g = torch.Generator(device=dev).manual_seed(0)
    q, k, v = (torch.randn(B, S, h, D, device=dev, generator=g).bfloat16().requires_grad_() for h in (H, Hk, Hk))
    go = torch.randn(B, S, H, D, device=dev, generator=g).bfloat16()
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    rows = {}

    def ours():
        return attention(q, k, v, causal=True, cu_seqlens=cu, window=args.window or None)

    rows["ours_fwd_ms"] = timed(lambda: ours(), args.iters, flush)
    if not args.no_backward:
        out = ours()
        rows["ours_bwd_ms"] = timed(lambda: torch.autograd.grad(out, (q, k, v), go, retain_graph=True), args.iters, flush)
    ops.check_status()
    if hasattr(ops.ext(), "attention_profile_read") and not args.no_backward:
        # a build with the backward kernel's cycle counters: one more backward, counters per query tile
        ops.ext().attention_profile_read(True)
        torch.autograd.grad(out, (q, k, v), go, retain_graph=True)
        torch.cuda.synchronize()
        c = ops.ext().attention_profile_read(True)
        tiles = max(c[0], 1)
        rows["bwd_cycles_per_query_tile"] = {i: round(c[i] / tiles, 1) for i in range(1, 16)}

    if not args.no_library and cu is None and not args.window:
        qh, kh, vh = (t.detach().transpose(1, 2).requires_grad_() for t in (q, k, v))

        def sdpa():
            return F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, enable_gqa=H != Hk)

        rows["sdpa_fwd_ms"] = timed(lambda: sdpa(), args.iters, flush)
        if not args.no_backward:
            o2 = sdpa()
            goh = go.transpose(1, 2)
            rows["sdpa_bwd_ms"] = timed(lambda: torch.autograd.grad(o2, (qh, kh, vh), goh, retain_graph=True),
                                        args.iters, flush)
    if not args.no_library:
        try:
            from flash_attn import flash_attn_func, flash_attn_varlen_func

            if cu is None:
                def fa():
                    return flash_attn_func(q, k, v, causal=True, window_size=(args.window - 1, 0) if args.window else (-1, -1))
            else:
                q3, k3, v3 = (t.detach()[0].requires_grad_() for t in (q, k, v))
                mx = max(lengths)

                def fa():
                    return flash_attn_varlen_func(q3, k3, v3, cu, cu, mx, mx, causal=True)

            rows["flash_attn2_fwd_ms"] = timed(lambda: fa(), args.iters, flush)
            if not args.no_backward:
                o3 = fa()
                ins = (q, k, v) if cu is None else (q3, k3, v3)
                g3 = go if cu is None else go[0]
                rows["flash_attn2_bwd_ms"] = timed(lambda: torch.autograd.grad(o3, ins, g3, retain_graph=True),
                                                   args.iters, flush)
        except Exception as exc:  # the wheel may lack sm_100 code
            rows["flash_attn2"] = f"unavailable: {type(exc).__name__}: {str(exc)[:120]}"
    for key in list(rows):
        if key.endswith("_fwd_ms"):
            rows[key.replace("_ms", "_tflops")] = flops_fwd / rows[key] / 1e9
        if key.endswith("_bwd_ms"):
            rows[key.replace("_ms", "_tflops")] = 2.5 * flops_fwd / rows[key] / 1e9
    rows["shape"] = dict(batch=B, seq=S, heads=H, kv_heads=Hk, dim=D, packed=args.packed, window=args.window)
    print(json.dumps(rows))
    return rows


if __name__ == "__main__":
    main()
