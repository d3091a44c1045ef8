"""`bench.py --metric ppo`: seconds per PPO iteration with four Llama-3.2-1B-style models.

This repository's arm is `benchmarks.bench_ppo_iter` (in-process paged-KV rollout, reward model
minus KL penalty, GAE, one PPO epoch in four minibatches with actor and critic sharded over the
ranks, weight hand-over to the engine every iteration) at 64 prompts of 256 tokens and 512
sampled tokens per rank: 512 prompts per 8-GPU box. The whole iteration is the public API path:
prompts start as host lists, sampled tokens and rewards come back to the host inside it, so the
device-timed value and the end-to-end value are the same measurement and both are reported from
separate sets of iterations.

The reference arm prints an `unavailable` line: the reference's PPO loop (scripts/ppo.py:230-420)
is tied to tokenised datasets, a tokenizer and text reward functions, and trains no critic
(projects/ppo/trainer.py has no value loss), so there is no stock code path that runs this
configuration on synthetic token data.
"""

from __future__ import annotations

import json
import os


def run(args):
    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({
                "impl": "reference", "metric": "PPO iteration time (4x Llama-3.2-1B-style models)",
                "unavailable": "the reference's PPO loop needs tokenised datasets, a tokenizer and text reward "
                               "functions (scripts/ppo.py:230-420) and has no critic update; no stock path runs the "
                               "synthetic 4-model configuration"}), flush=True)
        return
    from benchmarks import bench_ppo_iter
    from halite_b200.utils.timing import ClockSampler

    argv = ["--prompts", str(args.prompts_per_gpu), "--prompt-len", "256", "--new-tokens", str(args.new_tokens),
            "--minibatches", "4", "--iters", str(args.steps), "--warmup", str(args.warmup), "--quiet"]
    local = int(os.environ.get("LOCAL_RANK", "0"))
    with ClockSampler(local) as clocks:
        first = bench_ppo_iter.main(argv + ["--keep-group"])
        second = bench_ppo_iter.main(argv)
    if rank != 0:
        return
    world = first["n_gpus"]
    tokens = first["sampled_tokens_per_iteration_per_rank"]
    print(json.dumps({
        "metric": "PPO iteration time (4x Llama-3.2-1B-style models)", "value": first["value"], "unit": "s/iteration",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": first["value"] * 1e3,
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform-random prompts, random-init weights", "impl": "ours",
        "config": {"model": "llama-3.2-1b x4 (actor, critic, reference, reward)",
                   "prompts": args.prompts_per_gpu * world, "prompt_len": 256, "new_tokens": args.new_tokens,
                   "ppo": "GAE gamma 1.0 lambda 0.95, 1 epoch, 4 minibatches, clip 0.2, value clip 0.2, KL 0.05",
                   "parallelism": f"fsdp{world} actor + critic, one engine replica per GPU",
                   "l2": "four 1B models and the KV pool are larger than L2"},
        "e2e": {"value": second["value"], "unit": "s/iteration",
                "h2d_bytes_per_step": args.prompts_per_gpu * 256 * 8,
                "d2h_bytes_per_step": tokens * 8 + args.prompts_per_gpu * 4},
        "gpu_launches": first.get("gpu_launches", 0), "clocks": clocks.summary(),
        "phases_s_per_iteration": first["phases_s_per_iteration"],
        "peak_mem_gib": first.get("peak_mem_gib"),
    }), flush=True)
