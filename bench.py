"""Headline benchmark: Llama-3.2-3B pretraining step (bf16 compute, fp32 master weights and
AdamW, FSDP over N GPUs of one node), sequence length 4096, 8 sequences per GPU per step
(global batch 64 at 8 GPUs; weak scaling), synthetic uniform-random tokens, random-init weights.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref

Rank 0 prints ONE JSON line. `value` is whole-job tokens/s from CUDA-event time (max over
ranks) of exactly K steps; `e2e` repeats the measurement through the public training API
with a per-step pinned-host -> device copy of the tokens and a device -> host read of the loss.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL_NAME = "llama-3.2-3b"
SEQ_LEN = 4096
SEQS_PER_GPU = 8
VOCAB = 128256
# --model llama-3-8b is the second training configuration: tensor parallel 2 x FSDP 4 on 8 GPUs,
# sequence length 8192, global batch 32 (8 sequences per data-parallel rank, run as 2 micro-batches of 4)
TRAIN_MODELS = {
    "llama-3.2-3b": {"conf": "configs/models/llama/llama3_2_3b_bench.py", "dim": 3072, "label": "Llama-3.2-3B FSDP, seq 4096",
                     "tp": 1, "seq_len": 4096, "seqs_per_dp_rank": 8, "micro_batches": 1},
    "llama-3-8b": {"conf": "configs/models/llama/llama3_8b_bench.py", "dim": 4096, "label": "Llama-3-8B TP2 x FSDP, seq 8192",
                   "tp": 2, "seq_len": 8192, "seqs_per_dp_rank": 8, "micro_batches": 2},
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--metric", default="train", choices=["train", "rollout", "ppo"],
                    help="train: Llama-3.2-3B step (the headline); rollout: paged-KV decode tokens/s, one engine "
                         "replica per GPU; ppo: seconds per PPO iteration with four Llama-3.2-1B-style models")
    ap.add_argument("--requests-per-gpu", type=int, default=128, help="rollout: 1024 requests per 8-GPU box")
    ap.add_argument("--new-tokens", type=int, default=512)
    ap.add_argument("--prompts-per-gpu", type=int, default=64, help="ppo: 512 prompts per 8-GPU box")
    ap.add_argument("--model", default=MODEL_NAME, choices=sorted(TRAIN_MODELS),
                    help="train: llama-3.2-3b is the headline; llama-3-8b runs tensor parallel 2 x FSDP (gpus / 2)")
    ap.add_argument("--tp", type=int, default=None, help="train: tensor-parallel degree (default: the model's preset)")
    ap.add_argument("--micro-batches", type=int, default=None,
                    help="train: forward/backward passes per optimizer step (gradients accumulate, one reduction)")
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--seqs-per-gpu", type=int, default=None,
                    help="train: sequences per data-parallel rank and step (a rank is tp GPUs)")
    ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (marks the run invalid)")
    args = ap.parse_args()
    preset = TRAIN_MODELS[args.model]
    args.tp = args.tp or preset["tp"]
    args.seq_len = args.seq_len or preset["seq_len"]
    args.seqs_per_gpu = args.seqs_per_gpu or preset["seqs_per_dp_rank"]
    args.micro_batches = args.micro_batches or preset["micro_batches"]
    return args


def init_dist(n_gpus):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", local))
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    return rank, world, local


def make_batches(n, seqs, seq_len, rank, pinned=True):
    """n host batches of [seqs, seq_len + 1] uniform-random token ids (seeded per rank)."""
    import torch

    g = torch.Generator().manual_seed(1234 + rank)
    out = []
    for _ in range(n):
        t = torch.randint(0, VOCAB, (seqs, seq_len + 1), generator=g, dtype=torch.int64)
        out.append(t.pin_memory() if pinned else t)
    return out


def rollout_requests(args, rank, tag, warmup=False):
    """[(id, token ids, sampling params)] of one rank's share of a rollout batch: prompt lengths
    uniform in [128, 1024], uniform-random token ids, a quarter of the requests starting with one
    common 512-token prefix (the same on every rank), `--new-tokens` sampled tokens each at
    temperature 1.0 with EOS ignored. Warm-up batches are small (8 requests, 16 tokens)."""
    import random

    shared = random.Random(99).choices(range(VOCAB), k=512)
    rng = random.Random(hash((rank, tag)) & 0xffffffff)
    n_req = 8 if warmup else args.requests_per_gpu
    n_new = 16 if warmup else args.new_tokens
    out = []
    for i in range(n_req):
        n = rng.randint(128, 1024)
        ids = rng.choices(range(VOCAB), k=n)
        if rng.random() < 0.25:
            ids = shared + ids[: max(n - 512, 1)]
        out.append((f"{tag}-{rank}-{i}", ids,
                    {"max_new_tokens": n_new, "temperature": 1.0, "top_p": 1.0, "ignore_eos": True}))
    return out


def train_config(args, world):
    """`config` of a training record: identical in both arms for the same command line."""
    tp = args.tp
    dp = world // tp
    seqs, S, M = args.seqs_per_gpu, args.seq_len, args.micro_batches
    return {"model": args.model if not args.layers else f"{args.model}-{args.layers}layers-INVALID",
            "global_batch": seqs * dp, "seq_len": S, "micro_batches": M,
            "parallelism": f"fsdp{world}" if tp == 1 else f"tp{tp} x fsdp{dp}",
            "l2": f"inputs larger than L2 (activations of {seqs * S // M} tokens per pass)"}


def rollout_config(args, world):
    return {"model": MODEL_NAME, "requests": args.requests_per_gpu * world, "new_tokens": args.new_tokens,
            "prompt_len": "uniform [128, 1024], 25% share a 512-token prefix", "page_size": 16,
            "parallelism": f"dp{world} (one engine replica per GPU)", "sampling": "temperature 1.0, top-p 1.0, EOS ignored",
            "l2": "weights (6.4 GB) and KV pages are larger than L2"}


def run_rollout_ours(args):
    """Rollout decode throughput through the in-process paged-KV engine (`halite_b200.infer`)."""
    import torch
    import torch.distributed as dist

    rank, world, local = init_dist(args.gpus)
    dev = torch.device("cuda", local)

    from halite_b200 import ops
    from halite_b200.conf import instantiate, load_config
    from halite_b200.infer import InferenceEngine, InferenceRequest, ModelConfig, ServerConfig
    from halite_b200.utils.timing import ClockSampler, DeviceTimer

    C = ops.ext()
    conf = load_config(os.path.join(ROOT, "configs/models/llama/llama3_2_3b.py"))
    mc = conf.model_conf
    with torch.device("meta"):
        infer = instantiate(conf.model_infer)
        if callable(infer) and not isinstance(infer, torch.nn.Module):
            infer = instantiate(infer(conf.model))
    infer = infer.to(dtype=torch.bfloat16)
    infer.to_empty(device=dev)
    torch.manual_seed(0)
    infer.init_weights(dev)
    engine = InferenceEngine(
        infer, None,
        ModelConfig(n_heads=mc.n_heads, n_key_value_heads=mc.n_key_value_heads, head_dim=mc.head_dim,
                    n_layers=mc.n_layers, context_len=min(mc.context_len, 4096), device=f"cuda:{local}",
                    gpu_id=local, kv_cache_dtype=torch.bfloat16, vocab_size=mc.vocab_size, memory_fraction_static=0.8),
        ServerConfig(decode_steps_ahead=8, use_cudagraph=True))

    def to_requests(specs):
        return [InferenceRequest(i, ids, params) for i, ids, params in specs]

    W, K = args.warmup, args.steps
    for w in range(W):
        engine.infer_batch(to_requests(rollout_requests(args, rank, f"w{w}", warmup=True)))
    batches = [rollout_requests(args, rank, f"t{k}") for k in range(K)]
    e2e_batches = [rollout_requests(args, rank, f"e{k}") for k in range(K)]
    torch.cuda.synchronize()
    ops.check_status()
    new = e2e_new = h2d = d2h = 0
    C.reset_launch_count()
    with ClockSampler(local) as clocks:
        with DeviceTimer() as t:
            for specs in batches:
                for r in engine.infer_batch(to_requests(specs)):
                    new += len(r.output_ids[0])
        launches = C.launch_count()
        ms = t.max_ms()
        # end to end: prompts start in pinned host memory, results are read back as host lists
        with DeviceTimer() as te:
            for specs in e2e_batches:
                pinned = [torch.tensor(ids, dtype=torch.int64).pin_memory() for _, ids, _ in specs]
                reqs = [InferenceRequest(i, p.tolist(), params) for (i, _, params), p in zip(specs, pinned)]
                h2d += sum(p.numel() * 8 for p in pinned)
                for r in engine.infer_batch(reqs):
                    e2e_new += len(r.output_ids[0])
                    d2h += len(r.output_ids[0]) * 8
        e2e_ms = te.max_ms()
    ops.check_status()
    totals = torch.tensor([new, e2e_new], dtype=torch.float64, device=dev)
    if dist.is_initialized():
        dist.all_reduce(totals)
    if rank == 0:
        print(json.dumps({
            "metric": "rollout decode tokens/s (Llama-3.2-3B, paged KV, one replica per GPU)",
            "value": float(totals[0]) / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform-random prompts, random-init weights", "impl": "ours",
            "config": rollout_config(args, world),
            "e2e": {"value": float(totals[1]) / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / K,
                    "h2d_bytes_per_step": h2d // K, "d2h_bytes_per_step": d2h // K},
            "gpu_launches": int(launches), "clocks": clocks.summary(),
            "stack": "halite_b200.infer engine: paged prefill / decode kernels, tcgen05 GEMMs, CUDA-graph decode",
            "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30,
        }), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def run_ours(args):
    import torch
    import torch.distributed as dist

    if args.tp > 1 and args.gpus > args.tp:
        # the fused tensor-parallel GEMMs leave 20 SMs to the data-parallel collectives: keep NCCL within them
        os.environ.setdefault("NCCL_MAX_CTAS", "16")
    rank, world, local = init_dist(args.gpus)
    dev = torch.device("cuda", local)

    from halite_b200 import ops
    from halite_b200.conf import instantiate, load_config
    import contextlib

    from halite_b200.optim import build_optimizer, cycle_scheduler
    from halite_b200.optim.sharded_adamw import clip_grad_norm_
    from halite_b200.parallel import ParallelDims, parallelize
    from halite_b200.projects.common.train_fn import optimization_step
    from halite_b200.utils.timing import ClockSampler, DeviceTimer
    from functools import partial

    C = ops.ext()
    preset = TRAIN_MODELS[args.model]
    conf = load_config(os.path.join(ROOT, preset["conf"]))
    if args.layers:
        conf.model.blocks = conf.model.blocks[: args.layers]
    tp = args.tp
    if world % tp:
        raise SystemExit(f"--tp {tp} does not divide {world} GPUs")
    pd = ParallelDims(dp_replicate=1, dp_shard=world // tp, tp=tp, pp=1, world_size=world)
    pd.build_mesh("cuda")
    torch.manual_seed(0)
    with torch.device("meta"):
        model = instantiate(conf.model)
    model = parallelize(model, pd, pd, param_dtype="bfloat16", reduce_dtype="float32", device=dev)
    model.init_weights(dev)
    model._hb_fsdp.sync_parameters()
    optimizer = build_optimizer(partial(torch.optim.AdamW, lr=3e-4, betas=(0.9, 0.95), eps=1e-8), model,
                                weight_decay=0.1)
    scheduler = cycle_scheduler(optimizer, lr=3e-4, n_iter=10000, warmup=100)
    model.train()

    seqs, S, M = args.seqs_per_gpu, args.seq_len, args.micro_batches
    W, K = args.warmup, args.steps
    dp = world // tp
    # the ranks of one tensor-parallel group step on the same sequences
    host = make_batches(W + 2 * K + 2, seqs, S, pd.dp_rank if tp > 1 else rank)
    fsdp = model._hb_fsdp

    def step(tokens_dev):
        if M == 1:
            batch = {"input": tokens_dev[:, :-1], "target": tokens_dev[:, 1:]}
            return optimization_step(model, batch, optimizer, scheduler, clip_grad_norm=1.0,
                                    calc_loss_in_model=True)
        total = None
        for i, chunk in enumerate(tokens_dev.chunk(M)):
            # only the last micro-batch's backward starts the gradient reductions
            hold = fsdp.no_sync() if i < M - 1 else contextlib.nullcontext()
            with hold:
                loss = model(chunk[:, :-1], target=chunk[:, 1:]).loss / M
                loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        fsdp.finish_backward()
        clip_grad_norm_(model, 1.0, optimizer)
        scheduler.step()
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        return {"loss": total}

    # ---- warm-up (untimed)
    it = iter(host)
    for _ in range(W):
        out = step(next(it).to(dev, non_blocking=True))
    torch.cuda.synchronize()
    ops.check_status()

    # ---- device-timed region: inputs staged on the device beforehand
    staged = [next(it).to(dev) for _ in range(K)]
    C.reset_launch_count()
    with ClockSampler(local) as clocks:
        with DeviceTimer() as t:
            for i in range(K):
                out = step(staged[i])
        launches = C.launch_count()
        ms = t.max_ms()
        loss_dev = float(out["loss"].item())

        # ---- end-to-end through the public API: H2D of the step's tokens + D2H of its loss
        with DeviceTimer() as te:
            for i in range(K):
                tokens = next(it).to(dev, non_blocking=True)
                o = step(tokens)
                _ = float(o["loss"].item())
        e2e_ms = te.max_ms()
    ops.check_status()

    fused_units = [u for u in model._hb_fsdp.units if u.fused is not None]
    gather_mode = "none (one rank)" if world == 1 else "NCCL all-gather per unit, overlapped"
    if fused_units:
        carried = sum(u.fused.launches - u.fused.standalone for u in fused_units)
        heap = getattr(model._hb_fsdp, "reduce_heap", None)
        nvls = "yes" if heap is not None and heap.multicast_ptr and os.environ.get("HB_FSDP_NVLS", "1") != "0" else "no"
        gather_mode = (f"{len(fused_units)} block units: peers' shards copied over NVLink by CTAs inside GEMM launches "
                       f"({carried} carried, {sum(u.fused.standalone for u in fused_units)} launched alone so far); "
                       f"gradient reduction through NVLS multimem: {nvls}; root and head units: NCCL")
    tokens_per_step = seqs * S * dp
    value = tokens_per_step * K / (ms / 1e3)
    e2e = tokens_per_step * K / (e2e_ms / 1e3)
    n_params = sum(u.numel for u in model._hb_fsdp.units) * tp      # units hold this rank's tensor-parallel slice
    n_matmul = n_params - model.embedding.embed_weight.numel() * tp  # the embedding lookup is no GEMM
    flops_per_token = 6 * n_matmul + 6 * len(model.blocks) * S * preset["dim"]  # causal attention: 12*L*S*D/2
    peak_mem = torch.cuda.max_memory_allocated() / 2 ** 30
    if rank == 0:
        result = {
            "metric": f"train tokens/s ({preset['label']})", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform-random tokens, random-init weights",
            "impl": "ours",
            # the facts both arms share, under the same keys; what is specific to this arm sits in "arm"
            "config": train_config(args, world),
            "arm": {"optimizer": "AdamW fp32 master, clip 1.0",
                    "attention": "own tcgen05 kernels (forward + backward) inside the packed-QKV op",
                    "loss": "fused linear + cross entropy in the model", "fsdp_all_gather": gather_mode},
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": e2e_ms / K,
                    "h2d_bytes_per_step": seqs * (S + 1) * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "loss": loss_dev,
            "mfu_of_measured_sustained": None,
            "model_tflops_per_gpu": flops_per_token * tokens_per_step / world / (ms / K / 1e3) / 1e12,
            "peak_mem_gib": peak_mem,
        }
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
            result["mfu_of_measured_sustained"] = result["model_tflops_per_gpu"] / peaks["bf16_tflops_sustained"]
        except Exception:
            pass
        print(json.dumps(result), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse()
    if args.metric == "rollout":
        if args.impl == "reference":
            from baseline import reference_rollout

            reference_rollout.run(args)
        else:
            run_rollout_ours(args)
        return
    if args.metric == "ppo":
        from benchmarks import ppo_iteration

        ppo_iteration.run(args)
        return
    if args.impl == "reference":
        from baseline import reference_bench

        reference_bench.run(args)
        return
    run_ours(args)


if __name__ == "__main__":
    main()
