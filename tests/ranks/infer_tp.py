"""Rank script: the paged engine tensor-parallel over two Gloo ranks (CPU, fp32) against dense
decoding with the unsharded training model: greedy tokens equal, log-probs within 1e-4, weights of
each rank equal to slices of the full tensors."""

import os
from functools import partial

import torch
import torch.distributed as dist

from halite_b200.conf import instantiate
from halite_b200.conf.loader import load_module
from halite_b200.infer import InferenceEngine, InferenceRequest, ModelConfig, ServerConfig

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
zoo = load_module(os.path.join(ROOT, "configs/models/transformer.py"))
for split in (True, False):        # separate q / k / v + gate / up projections, then the packed forms
    kw = dict(vocab_size=1024, dim=256, n_heads=4, head_dim=64, n_layers=3, intermediate_size=688, context_len=512,
              n_key_value_heads=2, rms_norm_epsilon=1e-5, qkv_split=split, gated_ff_split=split,
              init=partial(torch.nn.init.normal_, std=0.02))
    cfg = zoo.transformer(**kw)
    torch.manual_seed(0)
    model = instantiate(cfg)
    model.init_weights()
    model.eval()
    with torch.device("meta"):
        imodel = instantiate(instantiate(zoo.transformer_infer(**kw, infer="paged"))(cfg))
    mc = ModelConfig(n_heads=4, n_key_value_heads=2, head_dim=64, n_layers=3, context_len=512, device="cpu",
                     kv_cache_dtype=torch.float32, tp_size=world)
    eng = InferenceEngine(imodel, None, mc, ServerConfig(max_total_tokens=4096, decode_steps_ahead=2))
    eng.load_state_dict(model.state_dict())
    assert eng.model_runner.kv_pool.kv_heads == 2 // world
    # every sharded tensor is the rank's slice of the full one
    full = model.state_dict()
    n_sharded = 0
    for k, v in imodel.state_dict().items():
        if tuple(v.shape) != tuple(full[k].shape):
            n_sharded += 1
            assert v.numel() * world == full[k].numel(), k
    assert n_sharded >= 3 * 4, n_sharded
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, 1024, (6, 24), generator=g).tolist()
    res = eng.infer_batch([InferenceRequest(i, p, {"max_new_tokens": 20, "top_k": 1, "n": 1}) for i, p in enumerate(prompts)])
    worst = 0.0
    for r in res:
        seq = torch.tensor([r.input_ids + r.output_ids[0]])
        with torch.no_grad():
            lp = torch.log_softmax(model(seq).logits[0].float(), -1)[len(r.input_ids) - 1:-1]
        assert lp.argmax(-1).tolist() == r.output_ids[0], (split, r.id)
        worst = max(worst, (lp.gather(-1, torch.tensor(r.output_ids[0])[:, None]).squeeze(-1)
                            - torch.tensor(r.output_logprobs[0])).abs().max().item())
    assert worst < 1e-4, worst
    # sampled (temperature 1) requests: both ranks must agree token for token
    res = eng.infer_batch([InferenceRequest(i, p, {"max_new_tokens": 12, "temperature": 1.0, "n": 2})
                           for i, p in enumerate(prompts[:3])])
    mine = torch.tensor([t for r in res for o in r.output_ids for t in o])
    both = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(both, mine)
    assert all(torch.equal(both[0], b) for b in both)
    print(f"TP_OK split={split} rank={rank} worst_logprob_diff={worst:.2e}")
dist.barrier()
dist.destroy_process_group()
