"""Model-zoo variants on CPU: a miniature Gemma-3-style multimodal decoder (vision tower, soft
image tokens, alternating local / global layers with per-type RoPE and bidirectional image
spans), Qwen3-style q/k norm with tied embeddings, SigLIP-style encoder, nGPT re-normalisation."""

import os
from functools import partial

import pytest
import torch
from torch import nn

from halite_b200.conf import instantiate
from halite_b200.conf.loader import load_module
from tests.helpers import ROOT

zoo = load_module(os.path.join(ROOT, "configs/models/transformer.py"))
init = partial(nn.init.normal_, std=0.05)


def build(cfg):
    torch.manual_seed(0)
    m = instantiate(cfg)
    m.init_weights()
    return m.eval()


def mini_gemma():
    from halite_b200.conf import load_config

    return load_config(os.path.join(ROOT, "tests/configs/mini_gemma3.py")).model


def test_mini_gemma3_multimodal_forward_and_masks():
    model = build(mini_gemma())
    keys = set(model.state_dict())
    assert "embedding.image_embedding.encoder.blocks.0.self_attention.module.q.bias" in keys
    assert "blocks.0.self_attention.post_norm.weight" in keys and "blocks.2.ff.post_norm.weight" in keys
    assert "embedding.text_embedding.multiplier" not in keys and not any(k.startswith("head.") for k in keys)
    ids = torch.randint(0, 98, (2, 12))
    ids[:, 3:7] = 99                               # one image = 4 soft tokens
    bid = torch.zeros(2, 12, dtype=torch.long)
    bid[:, 3:7] = 1
    images = torch.randn(2, 3, 16, 16)
    out = model(ids, images=images, bidirection_ids=bid)
    assert out.logits.shape == (2, 12, 100) and torch.isfinite(out.logits).all()
    # image tokens see each other both ways: changing the LAST image patch changes the logits at
    # the FIRST image position; text before the image is untouched (causal)
    images2 = images.clone()
    images2[:, :, 8:, 8:] += 1.0
    out2 = model(ids, images=images2, bidirection_ids=bid)
    assert (out2.logits[:, 3] - out.logits[:, 3]).abs().max() > 1e-4
    assert (out2.logits[:, :3] - out.logits[:, :3]).abs().max() < 1e-6
    # the bidirectional span is what lets position 3 see positions 4..6: without the ids the
    # logits there differ, while the last image position (which sees the whole span causally
    # anyway, window permitting) is a weaker check and text before the image never changes
    plain = model(ids, images=images)
    assert (plain.logits[:, 3] - out.logits[:, 3]).abs().max() > 1e-4
    assert (plain.logits[:, :3] - out.logits[:, :3]).abs().max() < 1e-6
    out.logits.float().mean().backward()


def test_qwen3_style_qk_norm_and_tied_head():
    from halite_b200.models.position import RotaryEmbedding, apply_rotary_emb
    from halite_b200.nn.normalization import RMSNorm

    cfg = zoo.transformer(vocab_size=64, dim=32, n_heads=4, head_dim=16, n_layers=2, intermediate_size=64,
                          context_len=32, n_key_value_heads=2, rms_norm_epsilon=1e-6,
                          pos_embed=RotaryEmbedding(16, 32, base=1000000, use_rotate_half=True, pre_init=False),
                          pos_embed_apply_fn=partial(apply_rotary_emb, use_complex=False), qkv_split=True,
                          gated_ff_split=True, q_norm=RMSNorm(16, eps=1e-6), k_norm=RMSNorm(16, eps=1e-6),
                          tie_embeds=True, init=init)
    model = build(cfg)
    sd = model.state_dict()
    assert "blocks.1.self_attention.module.attention.k_norm.weight" in sd and "head.linear.weight" not in sd
    x = torch.randint(0, 64, (2, 7))
    logits = model(x).logits
    assert logits.shape == (2, 7, 64)
    hidden = model(x, output_hidden_states=True).hidden_states[-1]
    torch.testing.assert_close(logits, hidden @ model.embedding.embed_weight.t(), rtol=1e-5, atol=1e-5)


def test_ngpt_normalize_projects_to_unit_rows():
    from halite_b200.models.optimizer import ngpt_normalize

    lin = nn.ModuleDict({"q": nn.Linear(8, 16, bias=True), "out": nn.Linear(16, 8, bias=False)})
    ngpt_normalize(lin)
    torch.testing.assert_close(lin["q"].weight.norm(dim=1), torch.ones(16))
    torch.testing.assert_close(lin["out"].weight.norm(dim=0), torch.ones(16))


def _train_a_little(model, vocab, post_step=None, steps=10, lr=3e-3):
    opt = torch.optim.AdamW(model.parameters(), lr=lr)
    x = torch.randint(0, vocab, (4, 17))
    losses = []
    for _ in range(steps):
        loss = torch.nn.functional.cross_entropy(model(x[:, :-1]).logits.flatten(0, 1).float(), x[:, 1:].flatten())
        loss.backward()
        opt.step()
        opt.zero_grad()
        if post_step is not None:
            post_step(model)
        losses.append(loss.item())
    return losses


def test_scaling_diff_transformer_and_ngpt_configs_train():
    from halite_b200.models.optimizer import ngpt_normalize

    torch.manual_seed(0)
    base = load_module(os.path.join(ROOT, "configs/models/scaling/base.py"))
    m = build(base.transformer(64, 32, 4, 8, 2, 48, 32, qkv_split=True, gated_ff_split=True, post_norm=True))
    m.train()
    losses = _train_a_little(m, 64)
    assert losses[-1] < losses[0] - 0.2

    diff = load_module(os.path.join(ROOT, "configs/models/diff_transformer.py"))
    m = build(diff.diff_transformer(64, 32, 2, 2, 48, 32, qkv_split=True))
    lam = [mod.lambda_init for mod in m.modules() if hasattr(mod, "lambda_init")]
    assert len(lam) == 2 and lam[0] == pytest.approx(0.2) and lam[1] > lam[0]
    m.train()
    losses = _train_a_little(m, 64)
    assert losses[-1] < losses[0] - 0.2

    ng = load_module(os.path.join(ROOT, "configs/models/ngpt.py"))
    m = build(ng.ngpt(64, 32, 4, 2, 48, 32))
    ngpt_normalize(m)
    m.train()
    losses = _train_a_little(m, 64, post_step=ngpt_normalize, lr=1e-2)
    assert losses[-1] < losses[0] - 0.1
    w = m.blocks["0"].self_attention.module.q.weight
    torch.testing.assert_close(w.norm(dim=1), torch.ones(32), rtol=1e-4, atol=1e-4)
    assert "blocks.0.self_attention.scale.weight" in m.state_dict()


def test_jit_and_diffusion_objectives():
    from halite_b200.projects.dit.diffusion import Diffusion, EquilibriumMatchingJiT

    jit = load_module(os.path.join(ROOT, "configs/models/jit.py"))
    model = build(jit.jit(image_size=16, patch_size=4, n_labels=10, dim=32, patch_dim=16, n_heads=2, head_dim=16,
                          n_layers=3, intermediate_size=64, in_context_len=2, in_context_start=1, qk_norm=True))
    x, lab = torch.randn(4, 3, 16, 16), torch.randint(0, 10, (4,))
    out = model(x, torch.rand(4), lab)
    assert out.shape == x.shape and out.abs().max() == 0          # adaLN-Zero: the head starts at zero
    assert "in_context_rope.freqs_cos" in model.state_dict() and "post_embed.linear.weight" in model.state_dict()
    d = Diffusion((3, 16, 16), 10, steps=4, guidance_scale=2.0, guidance_interval=(0.1, 1.0))

    def fixed_loss():
        torch.manual_seed(123)
        model.eval()
        v = sum(d.loss(model, x, lab).item() for _ in range(8)) / 8
        model.train()
        return v

    before = fixed_loss()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    torch.manual_seed(1)
    for _ in range(120):
        d.loss(model, x, lab).backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad()
    assert fixed_loss() < 0.7 * before
    model.eval()
    a, b = d.generate(model, lab, seed=1), d.generate(model, lab, seed=1)
    assert a.shape == x.shape and torch.equal(a, b) and torch.isfinite(a).all()
    # label dropping only while training; the unconditional id is n_labels
    d.train()
    d.label_drop_p = 1.0
    assert (d.drop_labels(lab) == 10).all()
    e = EquilibriumMatchingJiT((3, 16, 16), 10, steps=3, method="euler")
    t = torch.tensor([0.0, 0.8, 1.0]).view(-1, 1, 1, 1)
    assert e.get_c_t(t).flatten().tolist() == pytest.approx([4.0, 4.0, 0.0], abs=1e-5)
    assert torch.isfinite(e.loss(model, x, lab)) and e.generate(model, lab, seed=0).shape == x.shape


def test_encoder_jit_on_a_small_vision_encoder_and_its_unit_layout():
    """Encoder-JiT from its config builder on a tiny SigLIP-style encoder: forward shape, zero
    output at initialisation (adaLN-Zero head), frozen encoder, and one sharding unit per block
    of both block lists when wrapped with the block iterator."""
    from halite_b200.models.models.jit import encoder_jit_block_iterator
    from halite_b200.parallel import parallelize

    siglip = load_module(os.path.join(ROOT, "configs/models/siglip2/siglip_vision.py"))
    enc_jit = load_module(os.path.join(ROOT, "configs/models/encoder_jit.py"))
    encoder = build(zoo.transformer(**siglip.vision_config(32, 2, 2, 64, 16, 4)))
    wrap = instantiate(enc_jit.encoder_jit(image_size=16, patch_size=4, n_labels=10, dim=32, patch_dim=16, n_heads=2,
                                           head_dim=16, n_layers=3, intermediate_size=64, in_context_len=2,
                                           qk_norm=True, cond_start_id=1))
    model = wrap(encoder)
    model.init_weights("cpu")
    model.freeze_encoder()
    x, lab = torch.randn(2, 3, 16, 16), torch.randint(0, 10, (2,))
    out = model(x, torch.rand(2), lab)
    assert out.shape == x.shape and out.abs().max() == 0
    assert not any(p.requires_grad for p in model.encoder.parameters())
    model = parallelize(model, param_dtype="float32", reduce_dtype="float32", device="cpu",
                        block_iterator=encoder_jit_block_iterator)
    names = [u.name for u in model._hb_fsdp.units]
    assert names == ["root", "encoder.blocks.0", "encoder.blocks.1", "blocks.0", "blocks.1", "blocks.2"]
    assert model(x, torch.rand(2), lab).shape == x.shape
