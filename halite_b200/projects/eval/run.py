"""Generation-based evaluation on the paged engine (reference: scripts/eval_task.py:20-191).

Each task supplies a dataset, preprocessing to a `prompt` (and whatever its scorer needs), a
few-shot prefix, sampling parameters and an `evaluate_fn(record, [response]) -> {metric: value}`.
Prompts are sharded over data-parallel ranks; metric sums are reduced at the end.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from halite_b200.conf import instantiate
from halite_b200.data.dataset import MapDataset
from halite_b200.data.preprocess import Collator
from halite_b200.distributed.checkpoint import load_checkpoint
from halite_b200.infer.engine import InferenceEngine
from halite_b200.infer.types import ModelConfig
from halite_b200.utils import get_torch_dtype


def _get(c, k, d=None):
    return c.get(k, d) if hasattr(c, "get") else getattr(c, k, d)


def build_engine(model_conf, device="cuda", server_config=None, load=True):
    """`model_conf`: the `Model` section of a saved model folder."""
    with torch.device("meta"):
        infer = instantiate(model_conf.model_infer)
        if callable(infer) and not isinstance(infer, torch.nn.Module):
            infer = instantiate(infer(model_conf.model))
    mc = model_conf.model_conf
    dtype = get_torch_dtype(_get(mc, "dtype", "bfloat16")) if torch.device(device).type == "cuda" else torch.float32
    infer = infer.to(dtype=dtype)
    infer.to_empty(device=device)
    infer.eval()
    if load and model_conf.checkpoint_path is not None:
        load_checkpoint(infer, model_conf.checkpoint_path)
    tokenizer = instantiate(model_conf.tokenizer)
    return InferenceEngine(
        infer, tokenizer,
        ModelConfig(n_heads=_get(mc, "n_heads"), n_key_value_heads=_get(mc, "n_key_value_heads") or _get(mc, "n_heads"),
                    head_dim=_get(mc, "head_dim"), n_layers=_get(mc, "n_layers"), context_len=_get(mc, "context_len"),
                    kv_cache_dtype=dtype, device=torch.device(device).type, vocab_size=_get(mc, "vocab_size")),
        server_config)


def run_task(engine, task, eval_conf, logger=None, rank=0, world_size=1, max_batches=None):
    eval_fn = instantiate(task.evaluate_fn)
    ops = [instantiate(op) for op in (task.preprocess or [])]
    dset = MapDataset([instantiate(task.dataset)], [task.name], operations=ops)
    collate = Collator(())
    sampler = instantiate(task.fewshot.sampler)(instantiate(task.fewshot.samples)()) if task.fewshot is not None else None
    prefix_fn = instantiate(task.prefix) if task.prefix is not None else None
    tokenizer, limit = engine.tokenizer, engine.model_config.context_len
    totals, n = {}, 0
    indices = list(range(rank, len(dset), world_size))
    bs = eval_conf.batch_size
    for b, start in enumerate(range(0, len(indices), bs)):
        if max_batches is not None and b >= max_batches:
            break
        batch = collate([dset[i] for i in indices[start:start + bs]])
        requests = []
        for prompt in batch["prompt"]:
            prefix = prefix_fn(fewshot=sampler() if sampler is not None else None) if prefix_fn is not None else ""
            text = prefix + prompt
            ids = tokenizer.encode(text)
            params = task.sampling_params.build(len(ids), limit)
            requests.append({"id": len(requests), "input_ids": ids, "sampling_params": params})
        results = sorted(engine.infer_batch(requests), key=lambda r: r.id)
        for i, res in enumerate(results):
            response = tokenizer.decode(res.output_ids[0])
            metric = eval_fn(batch.slice(i), [response])
            for k, v in metric.items():
                totals[k] = totals.get(k, 0) + v
            n += 1
        if logger is not None:
            logger.info(f"{task.name} [{min(start + bs, len(indices))}/{len(indices)}]: " +
                        "; ".join(f"{k}: {v / max(n, 1):.4f}" for k, v in totals.items()))
    if world_size > 1 and dist.is_initialized():
        keys = sorted(totals)
        t = torch.tensor([totals[k] for k in keys] + [n], dtype=torch.float64)
        gathered = [None] * world_size
        dist.all_gather_object(gathered, t.tolist())
        summed = [sum(col) for col in zip(*gathered)]
        totals, n = dict(zip(keys, summed[:-1])), int(summed[-1])
    out = {k: v / max(n, 1) for k, v in totals.items()}
    out["n_samples"] = n
    return out
