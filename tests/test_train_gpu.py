"""End-to-end GPU checks: the kernel path of a small decoder against the PyTorch reference
path of the same weights, and the flagship smoke step."""

import os
from functools import partial

import pytest
import torch

pytestmark = pytest.mark.gpu


def _build(zoo, device, dtype_params="bfloat16", **over):
    from halite_b200.conf import instantiate
    from halite_b200.parallel import ParallelDims, parallelize
    from tests.conftest import tiny_llama_conf

    cfg = zoo.use_fused_linear_cross_entropy(tiny_llama_conf(zoo, **over))
    torch.manual_seed(0)
    with torch.device("meta"):
        model = instantiate(cfg)
    pd = ParallelDims(dp_shard=1, world_size=1)
    pd.build_mesh("cuda")
    model = parallelize(model, pd, pd, param_dtype=dtype_params, device=device)
    model.init_weights(device)
    return model


def test_kernel_path_matches_reference_path(zoo, monkeypatch):
    dev = torch.device("cuda", 0)
    model = _build(zoo, dev)
    tokens = torch.randint(0, 1024, (2, 129), device=dev)
    out = model(tokens[:, :-1], target=tokens[:, 1:])
    out.loss.backward()
    model._hb_fsdp.finish_backward()
    grads = [u.full_grad.clone() for u in model._hb_fsdp.units]
    for u in model._hb_fsdp.units:
        u._written.clear()
    monkeypatch.setenv("HALITE_B200_FORCE_REFERENCE", "1")
    out_r = model(tokens[:, :-1], target=tokens[:, 1:])
    out_r.loss.backward()
    model._hb_fsdp.finish_backward()
    assert abs(out.loss.item() - out_r.loss.item()) < 2e-2
    for g, u in zip(grads, model._hb_fsdp.units):
        ref = u.full_grad
        assert (g - ref).norm() / ref.norm().clamp(min=1e-6) < 5e-2


def test_smoke_entry():
    import __graft_entry__ as entry

    entry.smoke()


def test_loss_decreases_on_fixed_batch(zoo):
    from halite_b200.optim import build_optimizer
    from halite_b200.projects.common.train_fn import optimization_step

    dev = torch.device("cuda", 0)
    model = _build(zoo, dev)
    opt = build_optimizer(partial(torch.optim.AdamW, lr=1e-3, betas=(0.9, 0.95)), model, weight_decay=0.1)
    tokens = torch.randint(0, 1024, (4, 257), device=dev)
    losses = []
    for _ in range(8):
        out = optimization_step(model, {"input": tokens[:, :-1], "target": tokens[:, 1:]}, opt,
                               clip_grad_norm=1.0, calc_loss_in_model=True)
        losses.append(out["loss"].item())
    assert losses[-1] < losses[0] - 0.5, losses


def test_packed_varlen_path_matches_reference_path(zoo, monkeypatch):
    """Padding-free forward/backward (what the PPO trainer runs): kernels against the PyTorch
    reference path of the same weights, with the fused-residual block variant too."""
    from halite_b200.models.attention import build_unpad_params, unpad_input

    dev = torch.device("cuda", 0)
    for fused in (False, True):
        from halite_b200.conf import instantiate
        from halite_b200.parallel import ParallelDims, parallelize
        from tests.conftest import tiny_llama_conf

        cfg = tiny_llama_conf(zoo)
        if fused:
            cfg = zoo.use_fused_residual(cfg)
        torch.manual_seed(0)
        with torch.device("meta"):
            model = instantiate(cfg)
        pd = ParallelDims(dp_shard=1, world_size=1)
        pd.build_mesh("cuda")
        model = parallelize(model, pd, pd, param_dtype="bfloat16", device=dev)
        model.init_weights(dev)
        mask = torch.ones(3, 96, dtype=torch.int64, device=dev)
        mask[0, :17] = 0
        mask[2, :40] = 0                     # left padding, as in rollout batches
        tokens = torch.randint(0, 1024, (3, 96), device=dev)
        params = build_unpad_params(mask)
        ids = unpad_input(tokens.unsqueeze(-1), params).squeeze(-1)
        pos = unpad_input((mask.cumsum(1) - 1).clamp(min=0).unsqueeze(-1), params).squeeze(-1)

        def run():
            out = model(ids, position_ids=pos, unpad_params=params)
            loss = out.logits.float().log_softmax(-1)[..., :7].sum() / ids.numel()
            loss.backward()
            model._hb_fsdp.finish_backward()
            grads = [u.full_grad.clone() for u in model._hb_fsdp.units]
            for u in model._hb_fsdp.units:
                u._written.clear()
            return out.logits.detach().float(), grads

        logits, grads = run()
        monkeypatch.setenv("HALITE_B200_FORCE_REFERENCE", "1")
        logits_r, grads_r = run()
        monkeypatch.delenv("HALITE_B200_FORCE_REFERENCE")
        assert (logits - logits_r).abs().max() < 0.15
        for g, r in zip(grads, grads_r):
            assert (g - r).norm() / r.norm().clamp(min=1e-6) < 5e-2


def test_moe_decoder_trains_on_the_grouped_gemm_path():
    """A small mixture-of-experts decoder, sharded and in bf16, through the framework's update
    step: the expert layers run on the grouped GEMM modes and the loss goes down."""
    from halite_b200.conf import instantiate
    from halite_b200.conf.loader import load_module
    from halite_b200.nn.loss import CrossEntropyLoss
    from halite_b200.optim import build_optimizer
    from halite_b200.parallel import ParallelDims, parallelize
    from halite_b200.projects.common.train_fn import optimization_step

    dev = torch.device("cuda", 0)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    moe_zoo = load_module(os.path.join(root, "configs/models/moe_transformer.py"))
    cfg = moe_zoo.moe_transformer(vocab_size=512, dim=256, n_heads=4, n_layers=2, n_experts=8, expert_top_k=2,
                                  z_loss=1e-3, load_balance_loss=1e-2, intermediate_size=128,
                                  max_position_embeddings=128, qkv_split=True)
    torch.manual_seed(0)
    with torch.device("meta"):
        model = instantiate(cfg)
    pd = ParallelDims(dp_shard=1, world_size=1)
    pd.build_mesh("cuda")
    model = parallelize(model, pd, pd, param_dtype="bfloat16", device=dev)
    model.init_weights(dev)
    opt = build_optimizer(partial(torch.optim.AdamW, lr=2e-3, betas=(0.9, 0.95)), model, weight_decay=0.0)
    tokens = torch.randint(0, 512, (4, 129), device=dev)
    losses = []
    for _ in range(12):
        out = optimization_step(model, {"input": tokens[:, :-1], "target": tokens[:, 1:]}, opt,
                                criterion=CrossEntropyLoss(), clip_grad_norm=1.0)
        losses.append(float(out["loss_dict"]["cross entropy"]))
        assert "router-z-loss" in out["loss_dict"] or "load-balance-loss" in out["loss_dict"]
    assert losses[-1] < losses[0] - 0.5, losses


def test_hnet_runs_in_bf16_on_the_kernel_path():
    """Two-stage H-Net (Mamba-2 encoder / decoder blocks, attention main network) sharded in bf16:
    forward, ratio losses, backward and a few update steps on the GPU kernels."""
    from halite_b200.conf import instantiate, load_config
    from halite_b200.nn.loss import CrossEntropyLoss
    from halite_b200.optim import build_optimizer
    from halite_b200.parallel import ParallelDims, parallelize
    from halite_b200.projects.common.train_fn import optimization_step

    dev = torch.device("cuda", 0)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    conf = load_config(os.path.join(root, "configs/lm/hnet.py"), "stage2_tiny")
    torch.manual_seed(0)
    with torch.device("meta"):
        model = instantiate(conf.model.model)
    pd = ParallelDims(dp_shard=1, world_size=1)
    pd.build_mesh("cuda")
    model = parallelize(model, pd, pd, param_dtype="bfloat16", device=dev)
    model.init_weights(dev)
    opt = build_optimizer(partial(torch.optim.AdamW, lr=3e-3), model, weight_decay=0.0)
    pattern = torch.arange(64, device=dev) % 7
    ids = torch.stack([(pattern + k) % 256 for k in range(4)])
    losses = []
    for _ in range(20):
        out = optimization_step(model, {"input": ids[:, :-1], "target": ids[:, 1:]}, opt,
                                criterion=CrossEntropyLoss(), clip_grad_norm=1.0)
        losses.append(float(out["loss_dict"]["cross entropy"]))
        assert "ratio_loss" in out["loss_dict"]
    assert losses[-1] < 0.7 * losses[0], losses
