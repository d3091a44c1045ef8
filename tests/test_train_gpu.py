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
