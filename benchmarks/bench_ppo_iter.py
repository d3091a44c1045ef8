"""Time of one PPO iteration with four models (actor, critic, reference policy, reward model):

    python -m benchmarks.bench_ppo_iter [--prompts 64] [--prompt-len 256] [--new-tokens 512]
    torchrun --nproc-per-node N -m benchmarks.bench_ppo_iter ...      (FSDP over N ranks)

Per iteration and rank: push the actor's weights into the in-process paged engine, sample
`--new-tokens` tokens for `--prompts` random prompts, score them with the reward model (scalar
at the last token) minus a per-token KL penalty against the reference policy, GAE with the
critic's values, then one PPO epoch in `--minibatches` minibatches that updates the actor
(clipped surrogate) and the critic (clipped value loss), both sharded over the ranks with fp32
master AdamW. All four models share the Llama-3.2-1B architecture with random weights.
Prints one JSON line; the time is CUDA events around whole iterations, maximum over ranks.
"""

from __future__ import annotations

import argparse
import json
import os
import random
from functools import partial

import torch
import torch.distributed as dist


def _build(conf_node, pdims, device, wrapper=None, seed=0):
    from halite_b200.conf import instantiate

    with torch.device("meta"):
        model = instantiate(conf_node)
    if wrapper is not None:
        kwargs = {"device": device} if device.type == "cpu" else {}
        model = wrapper(model=model, mesh=pdims, parallel_dims=pdims, **kwargs)
    else:
        model.to_empty(device=device)
        if device.type == "cuda":
            model.to(torch.bfloat16)
    torch.manual_seed(seed)
    model.init_weights(device)
    return model


class PhaseTimer:
    """Device time per named phase, accumulated over iterations (CUDA events; wall clock on CPU)."""

    def __init__(self, device):
        self.cuda = device.type == "cuda"
        self.spans = []

    def span(self, name):
        timer = self

        class _Span:
            def __enter__(self):
                if timer.cuda:
                    self.a, self.b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    self.a.record()
                else:
                    import time

                    self.t0 = time.perf_counter()

            def __exit__(self, *exc):
                if timer.cuda:
                    self.b.record()
                    timer.spans.append((name, self.a, self.b))
                else:
                    import time

                    timer.spans.append((name, (time.perf_counter() - self.t0) * 1e3, None))

        return _Span()

    def totals(self):
        if self.cuda:
            torch.cuda.synchronize()
        out = {}
        self.each = {}
        for name, a, b in self.spans:
            ms = a.elapsed_time(b) if b is not None else a
            out[name] = out.get(name, 0.0) + ms
            self.each.setdefault(name, []).append(round(ms / 1e3, 4))
        self.spans = []
        return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--conf", default=None, help="model config (default: configs/models/llama/llama3_2_1b.py)")
    ap.add_argument("--prompts", type=int, default=64, help="prompts per rank (512 per 8-GPU box)")
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--new-tokens", type=int, default=512)
    ap.add_argument("--minibatches", type=int, default=4)
    ap.add_argument("--microbatch", type=int, default=16, help="sequences per forward/backward")
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--layers", type=int, default=0, help="keep only the first N blocks (0 = all)")
    ap.add_argument("--kl-coef", type=float, default=0.05)
    ap.add_argument("--resident-engine", action="store_true",
                    help="keep the engine's weights, KV pool and CUDA graphs on the device between rollouts "
                         "instead of freeing them for the training phases")
    ap.add_argument("--device", default=None)
    ap.add_argument("--quiet", action="store_true", help="return the result without printing it")
    ap.add_argument("--keep-group", action="store_true", help="leave the process group up for another call")
    args = ap.parse_args(argv)

    from halite_b200.conf import load_config
    from halite_b200.infer import InferenceEngine, ModelConfig, ServerConfig
    from halite_b200.optim import build_optimizer
    from halite_b200.optim.sharded_adamw import clip_grad_norm_
    from halite_b200.parallel import ParallelDims, parallelize
    from halite_b200.projects.common.rollout import Handler, RewardRegistry, Rollout, RolloutGenerator
    from halite_b200.projects.ppo.model import RewardModelScorer, ScalarHead, UnpaddedModel, ValueModel
    from halite_b200.projects.ppo.trainer import KLPenalty, PPOTrainer, compute_ppo_advantage
    from halite_b200.projects.ppo.train import clean_memory
    from halite_b200.projects.ppo.variants import PPOActorLoss

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev_type = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl" if dev_type == "cuda" else "gloo")
    pdims = ParallelDims(dp_replicate=1, dp_shard=world, tp=1, pp=1)
    device = torch.device(dev_type, pdims.local_rank) if dev_type == "cuda" else torch.device("cpu")
    if dev_type == "cuda":
        torch.cuda.set_device(device)
    pdims.build_mesh(dev_type)

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    conf = load_config(args.conf or os.path.join(root, "configs/models/llama/llama3_2_1b.py"))
    mc = conf.model_conf
    if args.layers:
        conf.model.blocks = conf.model.blocks[: args.layers]
        conf.model_body.blocks = conf.model_body.blocks[: args.layers]
    n_layers = args.layers or mc.n_layers
    dtype = "bfloat16" if dev_type == "cuda" else "float32"
    wrap = partial(parallelize, param_dtype=dtype, reduce_dtype="float32")

    actor = _build(conf.model, pdims, device, wrap, seed=0)
    critic_body = _build(conf.model_body, pdims, device, wrap, seed=1)
    ref = _build(conf.model, pdims, device, None, seed=0).requires_grad_(False)
    reward_body = _build(conf.model_body, pdims, device, None, seed=2).requires_grad_(False)
    value_head, reward_head = ScalarHead(mc.dim).to(device), ScalarHead(mc.dim).to(device)
    value_head.init_weights()
    reward_head.init_weights()
    if world > 1:
        for p in list(value_head.parameters()) + list(reward_head.parameters()):
            dist.broadcast(p.data, 0)
    critic = ValueModel(critic_body, value_head)
    reward_model = ValueModel(reward_body, reward_head)

    from halite_b200.conf import instantiate

    with torch.device("meta"):
        infer = instantiate(conf.model_infer)
        if callable(infer) and not isinstance(infer, torch.nn.Module):
            infer = instantiate(infer(conf.model))
    infer_dtype = torch.bfloat16 if dev_type == "cuda" else torch.float32
    infer = infer.to(dtype=infer_dtype)
    infer.to_empty(device=device)
    engine = InferenceEngine(
        infer, None,
        ModelConfig(n_heads=mc.n_heads, n_key_value_heads=mc.n_key_value_heads, head_dim=mc.head_dim,
                    n_layers=n_layers, context_len=args.prompt_len + args.new_tokens + 16, device=dev_type,
                    gpu_id=pdims.local_rank, kv_cache_dtype=infer_dtype, vocab_size=mc.vocab_size,
                    memory_fraction_static=0.5, distributed=False),
        ServerConfig(max_total_tokens=int(args.prompts * (args.prompt_len + args.new_tokens + 32) * 1.25),
                     use_cudagraph=dev_type == "cuda", decode_steps_ahead=8, keep_resident=args.resident_engine))
    timer = PhaseTimer(device)
    scorer = RewardModelScorer(reward_model, args.microbatch, device)

    def timed_scorer(input_ids, output_ids):
        with timer.span("reward_model"):
            return scorer(input_ids, output_ids)

    generator = RolloutGenerator(engine, RewardRegistry(
        Handler("reward_model", timed_scorer, args=("input_ids", "output_ids"))))

    trainer = PPOTrainer(
        actor=UnpaddedModel(actor), ref=UnpaddedModel(ref), critic=critic, device=device,
        advantage_fn=partial(compute_ppo_advantage, gamma=1.0, lam=0.95),
        actor_loss=PPOActorLoss(clip_low=0.2, clip_high=0.2, pg_loss_agg="token-mean"),
        penalty_fn=KLPenalty(args.kl_coef), log_probs_batch_size=args.microbatch, value_clip=0.2)
    adamw = partial(torch.optim.AdamW, lr=1e-6, betas=(0.9, 0.95))
    actor_opt = build_optimizer(adamw, actor, 0.0)
    critic_opt = build_optimizer(adamw, critic_body, 0.0)
    head_opt = torch.optim.AdamW(value_head.parameters(), lr=1e-5)

    rng = random.Random(1234 + rank)

    def make_prompts(tag):
        return [Rollout(id=f"{tag}-{rank}-{i}", input_ids=[rng.randrange(mc.vocab_size) for _ in range(args.prompt_len)],
                        type="bench", sampling_params={"max_new_tokens": args.new_tokens, "temperature": 1.0,
                                                       "top_p": 1.0, "ignore_eos": True})
                for i in range(args.prompts)]

    def iteration(tag):
        with timer.span("weight_sync"):
            clean_memory()
            generator.initialize()
            generator.load_state_dict(actor.state_dict())
        with timer.span("rollout_and_reward_model"):
            rollouts = generator.generate(make_prompts(tag))
        with timer.span("engine_release"):
            generator.cleanup()
            clean_memory()
        with timer.span("logprobs_values_gae"):
            rb = trainer.compute_advantage(rollouts)
        n_tokens = sum(len(r.output_ids) for r in rollouts)
        with timer.span("update"):
            size = (len(rollouts) + args.minibatches - 1) // args.minibatches
            for mb in rb.split(size):
                actor_opt.zero_grad(set_to_none=True)
                critic_opt.zero_grad(set_to_none=True)
                head_opt.zero_grad(set_to_none=True)
                micro = mb.split(args.microbatch)
                for m in micro:
                    res = trainer.compute_actor_loss(m)
                    (res.loss / len(micro)).backward()
                    closs, _ = trainer.compute_critic_loss(m)
                    (closs / len(micro)).backward()
                for model, opt in ((actor, actor_opt), (critic_body, critic_opt)):
                    fsdp = getattr(model, "_hb_fsdp", None)
                    if fsdp is not None:
                        fsdp.finish_backward()
                    clip_grad_norm_(model, 1.0, opt)
                    opt.step()
                if world > 1:
                    for p in value_head.parameters():
                        dist.all_reduce(p.grad)
                        p.grad /= world
                head_opt.step()
        return n_tokens

    for i in range(args.warmup):
        iteration(f"w{i}")
    timer.totals()
    if world > 1:
        dist.barrier()
    if dev_type == "cuda":
        torch.cuda.synchronize()
    import time

    t0 = time.perf_counter()
    a = b = None
    if dev_type == "cuda":
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
    tokens = 0
    for i in range(args.iters):
        tokens += iteration(f"t{i}")
    if dev_type == "cuda":
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
    else:
        ms = (time.perf_counter() - t0) * 1e3
    phases = timer.totals()
    stat = torch.tensor([ms] + [phases[k] for k in sorted(phases)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(stat, op=dist.ReduceOp.MAX)
    stat = stat.tolist()
    out = {"metric": "PPO iteration time", "value": stat[0] / 1e3 / args.iters, "unit": "s/iteration",
           "higher_is_better": False, "n_gpus": world, "iters": args.iters, "warmup": args.warmup,
           "prompts_per_rank": args.prompts, "prompt_len": args.prompt_len, "new_tokens": args.new_tokens,
           "minibatches": args.minibatches, "microbatch": args.microbatch, "layers": n_layers,
           "sampled_tokens_per_iteration_per_rank": tokens // args.iters,
           "phases_s_per_iteration": {k: round(v / 1e3 / args.iters, 4) for k, v in zip(sorted(phases), stat[1:])},
           "rollout_s_each_iteration_rank0": timer.each.get("rollout_and_reward_model"),
           "dtype": dtype, "data": "synthetic uniform-random prompts, random-init weights"}
    try:
        out["engine_stats"] = {k: (round(v, 3) if isinstance(v, float) else v) for k, v in dict(engine.stats).items()}
    except Exception:  # noqa: BLE001
        pass
    if dev_type == "cuda":
        out["peak_mem_gib"] = round(torch.cuda.max_memory_allocated() / 2 ** 30, 2)
    if dev_type == "cuda":
        from halite_b200 import ops

        out["gpu_launches"] = int(ops.ext().launch_count())
        ops.check_status()
    if rank == 0 and not args.quiet:
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        if not args.keep_group:
            dist.destroy_process_group()
    return out


if __name__ == "__main__":
    main()
