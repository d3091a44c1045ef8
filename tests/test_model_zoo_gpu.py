"""Model families on the GPU kernel path: each tiny variant is sharded in bf16, run forward and
backward on the sm_100a kernels and compared with the PyTorch reference path of the same weights."""

import os
from functools import partial

import pytest
import torch
from torch import nn

from tests.helpers import ROOT

pytestmark = pytest.mark.gpu
init = partial(nn.init.normal_, std=0.05)


def _wrap(cfg, dev):
    from halite_b200.conf import instantiate
    from halite_b200.parallel import ParallelDims, parallelize

    torch.manual_seed(0)
    with torch.device("meta"):
        model = instantiate(cfg)
    pd = ParallelDims(dp_shard=1, world_size=1)
    pd.build_mesh("cuda")
    model = parallelize(model, pd, pd, param_dtype="bfloat16", device=dev)
    model.init_weights(dev)
    return model


def _both_paths(model, monkeypatch, call):
    def run():
        logits = call(model)
        logits.float().square().mean().backward()
        model._hb_fsdp.finish_backward()
        grads = [u.full_grad.clone() for u in model._hb_fsdp.units]
        for u in model._hb_fsdp.units:
            u._written.clear()
        return logits.detach().float(), grads

    out, grads = run()
    monkeypatch.setenv("HALITE_B200_FORCE_REFERENCE", "1")
    out_r, grads_r = run()
    monkeypatch.delenv("HALITE_B200_FORCE_REFERENCE")
    assert torch.isfinite(out).all()
    scale = out_r.abs().max().clamp(min=1e-3)
    assert (out - out_r).abs().max() / scale < 5e-2, ((out - out_r).abs().max(), scale)
    for g, r in zip(grads, grads_r):
        assert (g - r).norm() / r.norm().clamp(min=1e-6) < 8e-2


def _families():
    from halite_b200.conf.loader import load_module
    from halite_b200.models.position import RotaryEmbedding, apply_rotary_emb
    from halite_b200.nn.normalization import RMSNorm

    zoo = load_module(os.path.join(ROOT, "configs/models/transformer.py"))
    base = load_module(os.path.join(ROOT, "configs/models/scaling/base.py"))
    diff = load_module(os.path.join(ROOT, "configs/models/diff_transformer.py"))
    ng = load_module(os.path.join(ROOT, "configs/models/ngpt.py"))
    yield "qwen3_style", zoo.transformer(
        vocab_size=256, dim=128, n_heads=4, head_dim=32, n_layers=2, intermediate_size=256, context_len=128,
        n_key_value_heads=2, rms_norm_epsilon=1e-6,
        pos_embed=RotaryEmbedding(32, 128, base=1000000, use_rotate_half=True, pre_init=False),
        pos_embed_apply_fn=partial(apply_rotary_emb, use_complex=False), qkv_split=True, gated_ff_split=True,
        q_norm=RMSNorm(32, eps=1e-6), k_norm=RMSNorm(32, eps=1e-6), tie_embeds=True, init=init)
    yield "scaling_post_norm_softcap", base.transformer(256, 128, 4, 32, 2, 256, 128, qkv_split=True,
                                                        gated_ff_split=True, post_norm=True, softcap=50.0)
    yield "diff_transformer", diff.diff_transformer(256, 128, 2, 2, 256, 128, qkv_split=True)
    yield "ngpt", ng.ngpt(256, 128, 4, 2, 256, 128)


@pytest.mark.parametrize("name", ["qwen3_style", "scaling_post_norm_softcap", "diff_transformer", "ngpt"])
def test_decoder_families_match_reference_path(name, monkeypatch):
    dev = torch.device("cuda", 0)
    cfg = dict(_families())[name]
    model = _wrap(cfg, dev)
    tokens = torch.randint(0, 256, (2, 64), device=dev)
    _both_paths(model, monkeypatch, lambda m: m(tokens).logits)


def test_mini_gemma3_multimodal_on_gpu(monkeypatch):
    from halite_b200.conf import load_config

    dev = torch.device("cuda", 0)
    model = _wrap(load_config(os.path.join(ROOT, "tests/configs/mini_gemma3.py")).model, dev)
    ids = torch.randint(0, 98, (2, 12), device=dev)
    ids[:, 3:7] = 99
    bid = torch.zeros(2, 12, dtype=torch.long, device=dev)
    bid[:, 3:7] = 1
    images = torch.randn(2, 3, 16, 16, device=dev, dtype=torch.bfloat16)
    _both_paths(model, monkeypatch, lambda m: m(ids, images=images, bidirection_ids=bid).logits)


def test_jit_diffusion_step_on_gpu():
    from halite_b200.conf.loader import load_module
    from halite_b200.projects.dit.diffusion import Diffusion

    dev = torch.device("cuda", 0)
    jit = load_module(os.path.join(ROOT, "configs/models/jit.py"))
    model = _wrap(jit.jit(image_size=32, patch_size=4, n_labels=10, dim=128, patch_dim=64, n_heads=4, head_dim=32,
                          n_layers=2, intermediate_size=256, in_context_len=4, in_context_start=1, qk_norm=True), dev)
    d = Diffusion((3, 32, 32), 10, steps=4, guidance_scale=2.0, guidance_interval=(0.1, 1.0))
    x = torch.randn(4, 3, 32, 32, device=dev, dtype=torch.bfloat16)
    lab = torch.randint(0, 10, (4,), device=dev)
    loss = d.loss(model, x, lab)
    loss.backward()
    model._hb_fsdp.finish_backward()
    assert torch.isfinite(loss) and all(torch.isfinite(u.full_grad).all() for u in model._hb_fsdp.units)
    model.eval()
    sample = d.generate(model, lab, seed=1)
    assert sample.shape == x.shape and torch.isfinite(sample.float()).all()
