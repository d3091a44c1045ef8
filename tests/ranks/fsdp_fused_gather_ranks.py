"""Launched by torchrun on >= 2 GPUs: trains a small decoder for a few steps twice from the same
seed, once with the parameter all-gather as a collective and once carried inside GEMM launches
over symmetric memory (then with the gradient reduce-scatter carried too), and checks that
losses and final parameters agree (the carrying GEMMs run on a different tile schedule and the
reduction adds the ranks in another order than the collective, so sums differ in the last bits)."""

import os
import sys
from functools import partial

import torch
import torch.distributed as dist


def main():
    from halite_b200 import ops
    from halite_b200.conf import instantiate
    from halite_b200.conf.loader import load_module
    from halite_b200.optim import build_optimizer
    from halite_b200.parallel import ParallelDims, parallelize
    from halite_b200.projects.common.train_fn import optimization_step

    dist.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    zoo = load_module(os.path.join(root, "configs/models/transformer.py"))
    cfg = zoo.use_fused_residual(zoo.use_fused_linear_cross_entropy(zoo.transformer(
        vocab_size=1024, dim=512, n_heads=8, head_dim=64, n_layers=4, intermediate_size=1408, context_len=256,
        n_key_value_heads=4, rms_norm_epsilon=1e-5, qkv_split=True, gated_ff_split=True,
        init=partial(torch.nn.init.normal_, std=0.02))))
    pd = ParallelDims(dp_shard=world)
    pd.build_mesh("cuda")
    torch.manual_seed(1 + rank)
    batches = [torch.randint(0, 1024, (4, 257), device=dev) for _ in range(5)]

    def train(fused, fused_reduce=False):
        torch.manual_seed(0)
        with torch.device("meta"):
            model = instantiate(cfg)
        model = parallelize(model, pd, pd, param_dtype="bfloat16", device=dev, fused_all_gather=fused,
                            fused_reduce_scatter=fused_reduce)
        model.init_weights(dev)
        model._hb_fsdp.sync_parameters()
        opt = build_optimizer(partial(torch.optim.AdamW, lr=1e-3, betas=(0.9, 0.95)), model, weight_decay=0.1)
        losses = []
        for tokens in batches:
            out = optimization_step(model, {"input": tokens[:, :-1], "target": tokens[:, 1:]}, opt,
                                    clip_grad_norm=1.0, calc_loss_in_model=True)
            losses.append(out["loss"].item())
        sd = {k: v.detach().clone() for k, v in model.state_dict().items()}
        torch.cuda.synchronize()
        ops.check_status()
        return losses, sd, model

    base_losses, base_sd, _ = train(False)
    losses, sd, model = train(True)
    units = [u for u in model._hb_fsdp.units if u.fused is not None]
    assert len(units) == 4, len(units)
    carried = sum(u.fused.launches - u.fused.standalone for u in units)
    alone = sum(u.fused.standalone for u in units)
    # per step: the first block's gather runs on its own, the other three ride on a GEMM;
    # the last step's gathers are flushed by state_dict()
    assert carried == 3 * 4 and alone == 4 + 4, (carried, alone)
    assert all(abs(a - b) < 2e-3 for a, b in zip(losses, base_losses)), (losses, base_losses)
    for k in base_sd:
        a, b = sd[k].float(), base_sd[k].float()
        assert (a - b).norm() <= 2e-2 * b.norm().clamp(min=1e-6), k
    # gradient reduce-scatter carried by backward GEMMs as well
    losses2, sd2, model2 = train(True, True)
    reducers = [u.fused_reduce for u in model2._hb_fsdp.units if u.fused_reduce is not None]
    assert len(reducers) == 4
    carried = sum(r.launches - r.standalone for r in reducers)
    alone = sum(r.standalone for r in reducers)
    assert carried == 3 * 5 and alone == 5, (carried, alone)     # per step: three ride, the first block's runs alone
    assert all(abs(a - b) < 2e-3 for a, b in zip(losses2, base_losses)), (losses2, base_losses)
    for k in base_sd:
        a, b = sd2[k].float(), base_sd[k].float()
        assert (a - b).norm() <= 2e-2 * b.norm().clamp(min=1e-6), k
    torch.cuda.synchronize()
    ops.check_status()
    dist.barrier()
    if rank == 0:
        print("RESULT ok", losses, losses2)
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
