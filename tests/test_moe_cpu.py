"""Mixture-of-experts: router semantics, expert layer against a per-token loop, the MoE decoder
config, and expert parallelism over Gloo ranks."""

import os

import pytest
import torch

from halite_b200.conf import instantiate
from halite_b200.conf.loader import load_module
from halite_b200.models.moe import (ExpertLinear, FeedForward, MoE, TopKRouter, expert_boundaries,
                                    top_k_softmax_with_capacity)
from halite_b200.models.moe.router import DROPPED
from halite_b200.nn.activation import SwiGLU
from tests.helpers import ROOT, run_ranks


def make_moe(E=4, k=2, d=16, h=24, **router):
    torch.manual_seed(0)
    m = MoE(TopKRouter(d, E, k, pre_softmax=True, deterministic=True, **router), None,
            FeedForward(ExpertLinear(E, d, 2 * h), SwiGLU(), ExpertLinear(E, h, d), top_k=k))
    for mod in m.modules():
        if hasattr(mod, "init_weights"):
            mod.init_weights()
    return m


def test_expert_layer_matches_per_token_loop_and_has_gradients():
    moe = make_moe(z_loss=1e-3, load_balance_loss=1e-2)
    x = torch.randn(3, 5, 16, requires_grad=True)
    y, aux = moe(x)
    assert set(aux) == {"router-z-loss", "load-balance-loss"}
    probs, idx, _ = moe.router(x)
    act, xf, ref = SwiGLU(), x.reshape(-1, 16), torch.zeros(15, 16)
    for t in range(15):
        for j in range(2):
            e = idx[t, j]
            ref[t] += probs[t, j] * (act(xf[t] @ moe.experts.linear1.weight[e]) @ moe.experts.linear2.weight[e])
    torch.testing.assert_close(y.reshape(-1, 16), ref, rtol=1e-5, atol=1e-6)
    (y.sum() + sum(aux.values())).backward()
    for p in (x, moe.experts.linear1.weight, moe.experts.linear2.weight, moe.router.gate.weight):
        assert p.grad is not None and p.grad.abs().sum() > 0
    # perfectly uniform routing gives a load-balance loss of exactly its coefficient
    moe.train()
    uniform = moe.router.calc_load_balance_loss(torch.zeros(8, 4), torch.full((4,), 4.0))
    assert uniform.item() == pytest.approx(1e-2)


def test_router_capacity_and_modes():
    torch.manual_seed(1)
    logits = torch.randn(16, 4)
    p, i, counts = top_k_softmax_with_capacity(logits, 2, pre_softmax=True, deterministic=True)
    assert counts.sum() == 32 and torch.equal(counts, torch.bincount(i.reshape(-1), minlength=4))
    p2, i2, _ = top_k_softmax_with_capacity(logits, 2, pre_softmax=False)
    torch.testing.assert_close(p2.sum(-1), torch.ones(16))
    pc, ic, before = top_k_softmax_with_capacity(logits, 2, capacity_factor=0.5, pre_softmax=True)
    kept = ic != DROPPED
    assert before.sum() == 32 and kept.sum() <= 4 * 4          # capacity = ceil(32 / 4 * 0.5) = 4 per expert
    assert (pc[~kept] == 0).all() and torch.bincount(ic[kept], minlength=4).max() <= 4
    pp, ip, _ = top_k_softmax_with_capacity(logits, 2, capacity_factor=0.5, pad_to_capacity=True, pre_softmax=True)
    assert pp.shape == (4, 4) and ip.shape == (4, 4)
    # dropped slots sort last and are excluded from the boundaries
    s, _ = ic.reshape(-1).sort()
    assert expert_boundaries(s, 4)[-1] == kept.sum()
    moe = make_moe(capacity_factor=0.5)
    y, _ = moe(torch.randn(2, 8, 16))
    assert torch.isfinite(y).all()


def test_moe_decoder_config_trains():
    zoo = load_module(os.path.join(ROOT, "configs/models/moe_transformer.py"))
    cfg = zoo.moe_transformer(vocab_size=64, dim=32, n_heads=4, n_layers=2, n_experts=4, expert_top_k=2, z_loss=1e-3,
                              load_balance_loss=1e-2, intermediate_size=48, max_position_embeddings=32,
                              qkv_split=True)
    torch.manual_seed(0)
    model = instantiate(cfg)
    model.init_weights()
    assert model.state_dict()["blocks.1.ff.module.experts.linear1.weight"].shape == (4, 32, 96)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    x = torch.randint(0, 64, (4, 17))
    first = None
    for _ in range(12):
        out = model(x[:, :-1])
        loss = torch.nn.functional.cross_entropy(out.logits.flatten(0, 1), x[:, 1:].flatten())
        aux = sum(v for a in out.aux_outputs if a for v in a.values())
        (loss + aux).backward()
        opt.step()
        opt.zero_grad()
        first = first or loss.item()
    assert loss.item() < first - 0.3 and float(aux) > 0


def test_expert_parallel_matches_single_process():
    outs = run_ranks(os.path.join(ROOT, "tests/ranks/moe_ep.py"), 2, timeout=300)
    assert all("RESULT" in o for o in outs), outs[0][-2000:]
