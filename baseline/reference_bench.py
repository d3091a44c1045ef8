"""Reference arm of bench.py.

Runs the UNMODIFIED reference package (installed with pip under `baseline/_ref`, its own
`configs/` tree copied beside it) for the same metric and config as the main arm: the
reference's `configs/models/llama/llama3_2_3b.py` model, its `parallelize()` (FSDP2 +
per-block torch.compile, bf16 params / fp32 reduce), its `CrossEntropyLoss`, its
`group_parameters` + torch AdamW, and the step order of its `scripts/lm.py` hot loop. None of
this repository's models, kernels or sharding layer is on that path; the only thing supplied
from here is the config-file loader, registered under the name of the reference's external
config dependency (which is not installable offline).

On one GPU the reference's `parallelize()` applies no sharding and therefore no bf16 mixed
precision; to keep the named precision regime the harness then calls the reference's own
`apply_compile` and `apply_fsdp` on a one-rank mesh (same functions, same arguments).
"""

from __future__ import annotations

import json
import os
import sys
import traceback

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
VOCAB = 128256


def _unavailable(reason: str):
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": reason.replace("\n", " ")[:300]}), flush=True)


def _model_config(name):
    """Path of the reference config file for `name`. The reference ships only the 3B file; the 8B one is
    that same file with the dimensions of Llama-3-8B substituted (written next to it so that its relative
    imports resolve), so the model is still built by the reference's own config code."""
    src = os.path.join(REF, "configs/models/llama/llama3_2_3b.py")
    if name == "llama-3.2-3b":
        return src
    text = open(src).read()
    for old, new in (("dim = 3072", "dim = 4096"), ("n_heads = 24", "n_heads = 32"), ("n_layers=28", "n_layers=32"),
                     ("intermediate_size=8192", "intermediate_size=14336")):
        if old not in text:
            raise RuntimeError(f"the reference's 3B config no longer contains {old!r}")
        text = text.replace(old, new)
    dst = os.path.join(REF, "configs/models/llama/llama3_8b.py")
    tmp = f"{dst}.{os.getpid()}.tmp"
    with open(tmp, "w") as f:
        f.write(text)
    os.replace(tmp, dst)
    return dst


def run(args):
    if not os.path.isdir(os.path.join(REF, "halite")):
        _unavailable("baseline/_ref/halite is missing (the reference was not installed with pip --target baseline/_ref)")
        return
    try:
        _run(args)
    except BaseException as e:  # noqa: BLE001
        traceback.print_exc(file=sys.stderr)
        _unavailable(f"reference run failed: {type(e).__name__}: {e}")


def _run(args):
    import torch
    import torch.distributed as dist
    from torch import nn

    sys.path.insert(0, ROOT)
    sys.path.insert(0, REF)
    import halite_b200.conf as hconf
    import halite_b200.conf.loader as hloader

    sys.modules.setdefault("slickconf", hconf)
    sys.modules.setdefault("slickconf.loader", hloader)
    from halite_b200.conf import instantiate, load_config
    from halite_b200.utils.timing import ClockSampler, DeviceTimer

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", "0")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)

    from halite.nn.loss import CrossEntropyLoss
    from halite.optim import group_parameters, lr_scheduler
    from halite.parallel import ParallelDims
    from halite.parallel.fsdp import apply_fsdp
    from halite.transformers.parallelize import apply_compile

    tp = getattr(args, "tp", 1) or 1
    M = getattr(args, "micro_batches", 1) or 1
    model_name = getattr(args, "model", "llama-3.2-3b")
    conf = load_config(_model_config(model_name))
    pdims = ParallelDims(dp_replicate=1, dp_shard=-1, tp=tp, pp=1)
    mesh = pdims.build_mesh("cuda")
    dp = world // tp
    dp_rank = rank // tp

    torch.manual_seed(0)
    with torch.device("meta"):
        model = instantiate(conf.model)
    if args.layers:
        for key in list(model.blocks._modules)[args.layers:]:
            del model.blocks._modules[key]
    if dp > 1:
        model = instantiate(conf.parallelize)(model=model, mesh=mesh, parallel_dims=pdims)
    elif tp > 1:
        # one data-parallel rank: the reference's mesh then has no dp dimension and its parallelize() would
        # skip sharding (and with it bf16 parameters); call its own apply_tp / apply_compile / apply_fsdp on a
        # (1, tp) mesh, as the one-GPU run does with a one-rank mesh
        from halite.transformers.parallelize import apply_tp
        from torch.distributed.device_mesh import init_device_mesh

        mesh2 = init_device_mesh("cuda", (1, tp), mesh_dim_names=("dp", "tp"))
        apply_tp(model, mesh2["tp"], None)
        apply_compile(model, None)
        apply_fsdp(model, mesh2["dp"], "bfloat16", "float32", True)
    else:
        # one GPU: the reference's parallelize() would apply no sharding and therefore no bf16 mixed
        # precision; call its own apply_compile and apply_fsdp on the one-rank mesh instead
        apply_compile(model, None)
        apply_fsdp(model, mesh["dp"], "bfloat16", "float32", True)
    model.to_empty(device=device)
    model.init_weights(device)

    fast = True
    try:
        import flash_attn.ops.triton.cross_entropy  # noqa: F401
    except Exception:
        fast = False
    criterion = CrossEntropyLoss(fast=fast)
    optimizer = torch.optim.AdamW(group_parameters(model, weight_decay=0.1), lr=3e-4, betas=(0.9, 0.95))
    scheduler = lr_scheduler.cycle_scheduler(optimizer, lr=3e-4, n_iter=10000, warmup=100)
    model.train()

    seqs, S, W, K = args.seqs_per_gpu, args.seq_len, args.warmup, args.steps
    g = torch.Generator().manual_seed(1234 + (dp_rank if tp > 1 else rank))
    host = [torch.randint(0, VOCAB, (seqs, S + 1), generator=g, dtype=torch.int64).pin_memory()
            for _ in range(W + 2 * K + 2)]

    def step(tokens):
        optimizer.zero_grad()
        total = None
        for i, chunk in enumerate(tokens.chunk(M)):
            # the reference's collator hands the loop separate contiguous input / target tensors
            inputs, labels = chunk[:, :-1].contiguous(), chunk[:, 1:].contiguous()
            if M > 1 and hasattr(model, "set_requires_gradient_sync"):
                model.set_requires_gradient_sync(i == M - 1)     # FSDP2: reduce once per optimizer step
            out = model(inputs)
            logits = out.logits
            if hasattr(logits, "full_tensor"):
                logits = logits.full_tensor()
            loss, _ = criterion(logits, labels)
            del out, logits
            if M > 1:
                loss = loss / M
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        loss = total
        nn.utils.clip_grad_norm_(model.parameters(), 1.0, foreach=True)
        scheduler.step()
        optimizer.step()
        return loss

    it = iter(host)
    for _ in range(W):
        loss = step(next(it).to(device, non_blocking=True))
    torch.cuda.synchronize()

    staged = [next(it).to(device) for _ in range(K)]
    with ClockSampler(local) as clocks:
        with DeviceTimer() as t:
            for i in range(K):
                loss = step(staged[i])
        ms = t.max_ms()
        loss_val = float(loss.item())
        with DeviceTimer() as te:
            for i in range(K):
                l = step(next(it).to(device, non_blocking=True))
                _ = float(l.item())
        e2e_ms = te.max_ms()

    from bench import train_config

    tokens_per_step = seqs * S * dp
    label = {"llama-3.2-3b": "Llama-3.2-3B FSDP, seq 4096", "llama-3-8b": "Llama-3-8B TP2 x FSDP, seq 8192"}[model_name]
    if rank == 0:
        print(json.dumps({
            "metric": f"train tokens/s ({label})",
            "value": tokens_per_step * K / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform-random tokens, random-init weights", "impl": "reference",
            "config": train_config(args, world),
            "arm": {"optimizer": "torch AdamW, clip 1.0", "attention": "SDPA (the reference's `torch` processor)",
                    "loss": f"CrossEntropyLoss(fast={fast}) on materialised logits",
                    "stack": "FSDP2 + torch.compile per block + SDPA + cuBLAS"},
            "e2e": {"value": tokens_per_step * K / (e2e_ms / 1e3), "unit": "tokens/s",
                    "ms_per_step": e2e_ms / K, "h2d_bytes_per_step": seqs * (S + 1) * 8,
                    "d2h_bytes_per_step": 4},
            "gpu_launches": 0,
            "clocks": clocks.summary(),
            "loss": loss_val,
            "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30,
        }), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
