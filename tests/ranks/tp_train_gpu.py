"""Launched by torchrun on >= 2 GPUs: tensor-parallel (x sharded data-parallel when there are more
than two ranks) bf16 training of a small decoder, once with the collectives inside the GEMM kernels
(all-gather -> GEMM, GEMM -> reduce-scatter over peer memory) and once with NCCL collectives beside
plain GEMMs, both against an fp32 single-process replica that steps on the same data."""

import os
from functools import partial

import torch
import torch.distributed as dist


def main():
    from halite_b200 import ops
    from halite_b200.conf import instantiate
    from halite_b200.conf.loader import load_module
    from halite_b200.optim import build_optimizer, group_parameters
    from halite_b200.optim.sharded_adamw import clip_grad_norm_
    from halite_b200.parallel import ParallelDims, parallelize

    dist.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    zoo = load_module(os.path.join(root, "configs/models/transformer.py"))

    def build(fused_head):
        cfg = zoo.transformer(vocab_size=1024, dim=512, n_heads=8, head_dim=64, n_layers=2, intermediate_size=1024,
                              context_len=256, n_key_value_heads=4, rms_norm_epsilon=1e-5, qkv_split=True,
                              gated_ff_split=True, init=partial(torch.nn.init.normal_, std=0.02))
        if fused_head:
            cfg = zoo.use_fused_linear_cross_entropy(cfg)
        torch.manual_seed(0)
        with torch.device(dev):
            m = instantiate(cfg)
        m.init_weights(dev)
        return m

    pd = ParallelDims(dp_shard=world // 2, tp=2)
    pd.build_mesh("cuda")
    dp, dp_rank = pd.dp, pd.dp_rank
    steps = 4
    g = torch.Generator().manual_seed(0)
    data = torch.randint(0, 1024, (dp, steps, 4, 257), generator=g).to(dev)

    def reference():
        ref = build(False).float()
        opt = torch.optim.AdamW(group_parameters(ref, 0.1), lr=1e-3, betas=(0.9, 0.95))
        losses = []
        for step in range(steps):
            tot = 0.0
            for r in range(dp):
                x = data[r, step]
                l = torch.nn.functional.cross_entropy(ref(x[:, :-1]).logits.float().flatten(0, 1),
                                                      x[:, 1:].flatten()) / dp
                l.backward()
                tot += l.item()
            torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
            opt.step()
            opt.zero_grad()
            losses.append(tot)
        return losses

    def train(async_tp):
        model = parallelize(build(True), pd, pd, param_dtype="bfloat16", reduce_dtype="float32", device=dev,
                            tensor_parallel_config={"enable_async_tp": async_tp})
        opt = build_optimizer(partial(torch.optim.AdamW, lr=1e-3, betas=(0.9, 0.95)), model, weight_decay=0.1)
        losses = []
        for step in range(steps):
            x = data[dp_rank, step]
            out = model(x[:, :-1], target=x[:, 1:])
            out.loss.backward()
            clip_grad_norm_(model, 1.0, opt)
            opt.step()
            opt.zero_grad()
            lt = out.loss.detach().float().clone()
            dist.all_reduce(lt)
            losses.append(lt.item() / world)
        torch.cuda.synchronize()
        ops.check_status()
        return losses, model

    ref_losses = reference()
    nccl_losses, _ = train(False)
    fused_losses, model = train(True)
    tp = model._hb_tp
    n_fused = len(tp._ag) + len(tp._rs)
    worst_nccl = max(abs(a - b) for a, b in zip(nccl_losses, ref_losses))
    worst_fused = max(abs(a - b) for a, b in zip(fused_losses, ref_losses))
    if rank == 0:
        print(f"ref {ref_losses}\nnccl {nccl_losses}\nfused {fused_losses} fused_ops={n_fused}")
    assert n_fused > 0, "the fused collective GEMMs did not run"
    assert worst_nccl < 3e-2 and worst_fused < 3e-2, (worst_nccl, worst_fused)
    dist.barrier()
    if rank == 0:
        print("RESULT ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
