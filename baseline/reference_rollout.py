"""Reference arm of `bench.py --metric rollout`.

Drives the UNMODIFIED reference package from `baseline/_ref`: its `transformer_infer` model
(`configs/models/llama/llama3_2_3b.py`, FlashInfer attention), its `InferenceEngine`, scheduler,
radix cache, memory pools and sampler, built the way its `scripts/ppo_monarch.py` builds them
(CUDA graphs on, extra graph sizes 1 / 2 / 4 / 8), on the request mix of the main arm: one engine
replica per GPU, each with the same number of requests. Nothing of this repository's engine or
kernels is on that path; only the config-file loader comes from here (registered under the name
of the reference's external config dependency, which cannot be installed offline).
"""

from __future__ import annotations

import json
import os
import sys
import traceback

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def _unavailable(reason: str, metric: str):
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "metric": metric,
                          "unavailable": " ".join(str(reason).split())[:400]}), flush=True)


def run(args):
    metric = "rollout decode tokens/s (Llama-3.2-3B, paged KV, one replica per GPU)"
    if not os.path.isdir(os.path.join(REF, "halite")):
        _unavailable("baseline/_ref/halite is missing (the reference was not installed with pip --target baseline/_ref)",
                     metric)
        return
    try:
        _run(args, metric)
    except BaseException as e:  # noqa: BLE001
        traceback.print_exc(file=sys.stderr)
        _unavailable(f"reference rollout failed: {type(e).__name__}: {e}", metric)


def _run(args, metric):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    sys.path.insert(0, REF)
    import halite_b200.conf as hconf
    import halite_b200.conf.loader as hloader

    sys.modules.setdefault("slickconf", hconf)
    sys.modules.setdefault("slickconf.loader", hloader)
    from halite_b200.conf import instantiate, load_config
    from halite_b200.utils.timing import ClockSampler, DeviceTimer

    from bench import init_dist, rollout_requests       # the request mix is shared by both arms

    rank, world, local = init_dist(args.gpus)
    device = torch.device("cuda", local)

    from halite.transformers.infer import InferenceEngine, ModelConfig
    from halite.transformers.infer.types import InferenceRequest, ServerConfig

    conf = load_config(os.path.join(REF, "configs/models/llama/llama3_2_3b.py"))
    mc = conf.model_conf
    with torch.device("meta"):
        infer = instantiate(conf.model_infer)
        if callable(infer) and not isinstance(infer, torch.nn.Module):
            infer = instantiate(infer(conf.model))
    infer = infer.to(dtype=torch.bfloat16)
    infer.to_empty(device=device)
    torch.manual_seed(0)
    with torch.no_grad():
        for p in infer.parameters():
            torch.nn.init.normal_(p, std=0.02)
        for name, p in infer.named_parameters():
            if p.ndim == 1 and "norm" in name:
                p.fill_(1.0)
    engine = InferenceEngine(
        infer, None,
        ModelConfig(n_heads=mc.n_heads, n_key_value_heads=mc.n_key_value_heads, head_dim=mc.head_dim,
                    n_layers=mc.n_layers, context_len=min(mc.context_len, 4096), memory_fraction_static=0.8,
                    kv_cache_dtype=torch.bfloat16, gpu_id=local, distributed=False),
        ServerConfig(use_cudagraph=True, cudagraph_additonal_batch_size=(1, 2, 4, 8)))

    def to_requests(specs):
        return [InferenceRequest(i, ids, params) for i, ids, params in specs]

    W, K = args.warmup, args.steps
    for w in range(W):
        engine.infer_batch(to_requests(rollout_requests(args, rank, f"w{w}", warmup=True)))
    batches = [rollout_requests(args, rank, f"t{k}") for k in range(K)]
    e2e_batches = [rollout_requests(args, rank, f"e{k}") for k in range(K)]
    new = prompt = 0
    with ClockSampler(local) as clocks:
        with DeviceTimer() as t:
            for specs in batches:
                for r in engine.infer_batch(to_requests(specs)):
                    new += len(r.output_ids[0])
                    prompt += len(r.input_ids)
        ms = t.max_ms()
        e2e_new = 0
        h2d = d2h = 0
        with DeviceTimer() as te:
            for specs in e2e_batches:
                pinned = [torch.tensor(ids, dtype=torch.int64).pin_memory() for _, ids, _ in specs]
                reqs = [InferenceRequest(i, p.tolist(), params) for (i, _, params), p in zip(specs, pinned)]
                h2d += sum(p.numel() * 8 for p in pinned)
                for r in engine.infer_batch(reqs):
                    e2e_new += len(r.output_ids[0])
                    d2h += len(r.output_ids[0]) * 8
        e2e_ms = te.max_ms()
    totals = torch.tensor([new, e2e_new], dtype=torch.float64, device=device)
    if dist.is_initialized():
        dist.all_reduce(totals)
    if rank == 0:
        print(json.dumps({
            "metric": metric, "value": float(totals[0]) / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform-random prompts, random-init weights", "impl": "reference",
            "config": rollout_config(args, world),
            "e2e": {"value": float(totals[1]) / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / K,
                    "h2d_bytes_per_step": h2d // K, "d2h_bytes_per_step": d2h // K},
            "gpu_launches": 0, "clocks": clocks.summary(),
            "stack": "reference InferenceEngine + FlashInfer backend + CUDA graphs",
            "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30,
        }), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def rollout_config(args, world):
    from bench import rollout_config as shared

    return shared(args, world)
