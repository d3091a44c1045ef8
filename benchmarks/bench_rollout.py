"""Rollout throughput of one engine replica:

    python -m benchmarks.bench_rollout [--requests 128] [--new-tokens 512] [--engine paged|tokainfer]

Llama-3.2-3B architecture with random bf16 weights; prompt lengths uniform in [min, max] with
uniform-random token ids, a share of the requests starting with one common 512-token prefix
(exercises the prefix cache); temperature 1.0, EOS ignored. A box runs one replica per GPU, so
box throughput is this number times the GPU count. Prints one JSON line; times are device
events around the whole `infer_batch` call (host scheduling included).
"""

from __future__ import annotations

import argparse
import json
import os
import random

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--conf", default=None)
    ap.add_argument("--requests", type=int, default=128)
    ap.add_argument("--min-prompt", type=int, default=128)
    ap.add_argument("--max-prompt", type=int, default=1024)
    ap.add_argument("--new-tokens", type=int, default=512)
    ap.add_argument("--shared-frac", type=float, default=0.25)
    ap.add_argument("--shared-len", type=int, default=512)
    ap.add_argument("--engine", default="paged", choices=["paged", "tokainfer"])
    ap.add_argument("--layers", type=int, default=0, help="keep only the first N blocks (0 = all)")
    ap.add_argument("--warmup-requests", type=int, default=8)
    ap.add_argument("--steps-ahead", type=int, default=8)
    ap.add_argument("--no-cudagraph", action="store_true")
    ap.add_argument("--profile", type=int, default=0, help="print the top N kernels by device time (slows the run)")
    args = ap.parse_args(argv)

    from halite_b200.conf import instantiate, load_config
    from halite_b200.infer import InferenceRequest, ModelConfig

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    conf = load_config(args.conf or os.path.join(root, "configs/models/llama/llama3_2_3b.py"))
    mc = conf.model_conf
    model_conf = conf.model
    if args.layers:
        model_conf.blocks = model_conf.blocks[: args.layers]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    with torch.device("meta"):
        infer = instantiate(conf.model_infer)
        if callable(infer) and not isinstance(infer, torch.nn.Module):
            infer = instantiate(infer(model_conf))
    infer = infer.to(dtype=torch.bfloat16)
    infer.to_empty(device=dev)
    torch.manual_seed(0)
    infer.init_weights(dev)
    n_layers = args.layers or mc.n_layers
    model_config = ModelConfig(n_heads=mc.n_heads, n_key_value_heads=mc.n_key_value_heads, head_dim=mc.head_dim,
                               n_layers=n_layers, context_len=min(mc.context_len, 4096), device="cuda",
                               kv_cache_dtype=torch.bfloat16, vocab_size=mc.vocab_size, memory_fraction_static=0.8)
    if args.engine == "paged":
        from halite_b200.infer import InferenceEngine, ServerConfig

        engine = InferenceEngine(infer, None, model_config,
                                 ServerConfig(decode_steps_ahead=args.steps_ahead, use_cudagraph=not args.no_cudagraph))
    else:
        from halite_b200.tokainfer import InferenceEngine, ServerConfig

        engine = InferenceEngine(infer, None, model_config, ServerConfig(scheduling_steps_ahead=args.steps_ahead,
                                                                        memory_fraction=0.8))
    rng = random.Random(0)
    shared = [rng.randrange(mc.vocab_size) for _ in range(args.shared_len)]

    def make(i, n_new):
        n = rng.randint(args.min_prompt, args.max_prompt)
        ids = [rng.randrange(mc.vocab_size) for _ in range(n)]
        if rng.random() < args.shared_frac:
            ids = shared + ids[: max(n - args.shared_len, 1)]
        return InferenceRequest(i, ids, {"max_new_tokens": n_new, "temperature": 1.0, "top_p": 1.0, "ignore_eos": True})

    engine.infer_batch([make(f"w{i}", 16) for i in range(args.warmup_requests)])      # warm-up: graphs, caches
    reqs = [make(i, args.new_tokens) for i in range(args.requests)]
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    prof = None
    if args.profile:
        from torch.profiler import ProfilerActivity, profile

        prof = profile(activities=[ProfilerActivity.CUDA])
        prof.__enter__()
    start.record()
    results = engine.infer_batch(reqs)
    end.record()
    torch.cuda.synchronize()
    if prof is not None:
        prof.__exit__(None, None, None)
        rows = sorted(((e.key, e.device_time_total, e.count) for e in prof.key_averages() if e.device_time_total > 0),
                      key=lambda r: -r[1])
        total = sum(r[1] for r in rows)
        print(f"{total / 1e3:.1f} ms of kernels")
        for name, t, n in rows[: args.profile]:
            print(f"{100 * t / total:6.2f}% {t / 1e3:9.2f} ms {n:7d}  {name[:100]}")
    ms = start.elapsed_time(end)
    new = sum(len(r.output_ids[0]) for r in results)
    prompt = sum(len(r.input_ids) for r in results)
    cached = sum(r.num_cached_prompt_tokens[0] or 0 for r in results)
    out = {"metric": "rollout decode tokens/s per replica", "engine": args.engine, "value": new / ms * 1e3,
           "unit": "tokens/s", "requests": len(results), "new_tokens": new, "prompt_tokens": prompt,
           "cached_prompt_tokens": cached, "seconds": ms / 1e3, "total_tokens_per_s": (new + prompt - cached) / ms * 1e3,
           "layers": n_layers, "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30}
    try:
        out["engine_stats"] = {k: (round(v, 3) if isinstance(v, float) else v) for k, v in dict(engine.stats).items()}
    except Exception:  # noqa: BLE001
        pass
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
