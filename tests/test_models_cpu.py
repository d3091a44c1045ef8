import math
from functools import partial

import pytest
import torch

from halite_b200.conf import instantiate
from tests.conftest import tiny_llama_conf


def test_state_dict_keys_match_reference_format(zoo):
    model = instantiate(tiny_llama_conf(zoo, n_layers=2))
    keys = set(model.state_dict().keys())
    expect = {
        "embedding.embed_input_ids.weight", "post_blocks.module.weight", "head.linear.weight",
        "blocks.0.self_attention.pre_norm.weight", "blocks.0.self_attention.module.q.weight",
        "blocks.0.self_attention.module.k.weight", "blocks.0.self_attention.module.v.weight",
        "blocks.0.self_attention.module.out.weight", "blocks.0.ff.pre_norm.weight",
        "blocks.0.ff.module.linear_proj.weight", "blocks.0.ff.module.linear_gate.weight",
        "blocks.0.ff.module.linear_out.weight",
    }
    assert expect <= keys
    fused = instantiate(tiny_llama_conf(zoo, n_layers=1, qkv_split=False, gated_ff_split=False))
    k2 = set(fused.state_dict().keys())
    assert {"blocks.0.self_attention.module.qkv.weight", "blocks.0.ff.module.linear1.weight",
            "blocks.0.ff.module.linear2.weight"} <= k2


def test_tied_embeddings_drop_head_key(zoo):
    model = instantiate(tiny_llama_conf(zoo, n_layers=1, tie_embeds=True))
    sd = model.state_dict()
    assert "head.linear.weight" not in sd
    assert model.head.linear.weight is model.embedding.embed_input_ids.weight
    other = instantiate(tiny_llama_conf(zoo, n_layers=1, tie_embeds=True))
    other.load_state_dict(sd)
    x = torch.randint(0, 1024, (1, 8))
    assert torch.allclose(model(x).logits, other(x).logits)


def test_forward_matches_handwritten_llama(zoo):
    """Decoder output against a direct restatement of the Llama block equations."""
    torch.manual_seed(0)
    model = instantiate(tiny_llama_conf(zoo, n_layers=2))
    model.init_weights()
    sd = model.state_dict()
    x = torch.randint(0, 1024, (2, 24))
    got = model(x).logits

    def rms(h, w):
        return h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5) * w

    H, Hk, D = 4, 2, 64
    h = sd["embedding.embed_input_ids.weight"][x]
    S = x.shape[1]
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.arange(S).float()[:, None] * inv[None]
    cos, sin = ang.cos()[None, :, None], ang.sin()[None, :, None]

    def rope(t):
        a, b = t[..., 0::2], t[..., 1::2]
        return torch.stack((a * cos - b * sin, a * sin + b * cos), -1).flatten(-2)

    for i in range(2):
        p = f"blocks.{i}."
        n = rms(h, sd[p + "self_attention.pre_norm.weight"])
        q = (n @ sd[p + "self_attention.module.q.weight"].t()).view(2, S, H, D)
        k = (n @ sd[p + "self_attention.module.k.weight"].t()).view(2, S, Hk, D)
        v = (n @ sd[p + "self_attention.module.v.weight"].t()).view(2, S, Hk, D)
        q, k = rope(q), rope(k)
        k = k.repeat_interleave(H // Hk, 2)
        v = v.repeat_interleave(H // Hk, 2)
        s = torch.einsum("bqhd,bkhd->bhqk", q, k) / math.sqrt(D)
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
        a = torch.einsum("bhqk,bkhd->bqhd", s.softmax(-1), v).reshape(2, S, H * D)
        h = h + a @ sd[p + "self_attention.module.out.weight"].t()
        n = rms(h, sd[p + "ff.pre_norm.weight"])
        up = n @ sd[p + "ff.module.linear_proj.weight"].t()
        gate = n @ sd[p + "ff.module.linear_gate.weight"].t()
        h = h + (up * torch.nn.functional.silu(gate)) @ sd[p + "ff.module.linear_out.weight"].t()
    want = rms(h, sd["post_blocks.module.weight"]) @ sd["head.linear.weight"].t()
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-4)


def test_llama3_rope_scaling_bands():
    from halite_b200.models.position import Llama3RoPE, RotaryEmbedding

    plain = RotaryEmbedding(128, 8192, base=500000).inv_freq
    scaled = Llama3RoPE(128, 8192, use_scaled_rope=True, scale_factor=32).inv_freq
    wavelen = 2 * math.pi / plain
    hi = wavelen < 8192 / 4
    lo = wavelen > 8192 / 1
    assert torch.allclose(scaled[hi], plain[hi])
    assert torch.allclose(scaled[lo], plain[lo] / 32)
    mid = ~(hi | lo)
    assert mid.any() and (scaled[mid] < plain[mid]).all() and (scaled[mid] > plain[mid] / 32 / 32).all()


def test_rope_modes_agree_with_complex_multiply():
    from halite_b200.models.position import RotaryEmbedding, apply_rotary_emb

    torch.manual_seed(0)
    q = torch.randn(2, 10, 4, 64)
    k = torch.randn(2, 10, 2, 64)
    pos = torch.arange(10).unsqueeze(0)
    inter = RotaryEmbedding(64, 128, use_complex=True)
    table = inter(pos, 10, None, q.device, q.dtype)
    q1, k1 = apply_rotary_emb(q, k, table, use_complex=True)
    freqs = torch.outer(torch.arange(10).float(), inter.inv_freq)
    cis = torch.polar(torch.ones_like(freqs), freqs)[None, :, None]
    qc = torch.view_as_real(torch.view_as_complex(q.reshape(2, 10, 4, 32, 2)) * cis).flatten(-2)
    assert torch.allclose(q1, qc, atol=1e-5)
    half = RotaryEmbedding(64, 128, use_rotate_half=True)
    q2, _ = apply_rotary_emb(q, k, half(pos, 10, None, q.device, q.dtype))
    cos = torch.cat((freqs.cos(), freqs.cos()), -1)[None, :, None]
    sin = torch.cat((freqs.sin(), freqs.sin()), -1)[None, :, None]
    rot = torch.cat((-q[..., 32:], q[..., :32]), -1)
    assert torch.allclose(q2, q * cos + rot * sin, atol=1e-5)


def test_kv_cache_generation_matches_full_forward(zoo):
    torch.manual_seed(0)
    model = instantiate(tiny_llama_conf(zoo, n_layers=2)).eval()
    model.init_weights()
    x = torch.randint(0, 1024, (2, 12))
    full = model(x).logits
    out = model(x[:, :8], use_cache=True)
    cache = out.cache
    logits = [out.logits]
    for t in range(8, 12):
        out = model(x[:, t:t + 1], cache=cache, use_cache=True)
        cache = out.cache
        logits.append(out.logits)
    assert torch.allclose(torch.cat(logits, 1), full, atol=1e-4)


def test_fused_linear_ce_head_matches_criterion(zoo):
    from halite_b200.nn.loss import CrossEntropyLoss

    torch.manual_seed(0)
    base = tiny_llama_conf(zoo, n_layers=1)
    model = instantiate(base)
    model.init_weights()
    fused = instantiate(zoo.use_fused_linear_cross_entropy(base, z_loss=1e-4))
    fused.load_state_dict(model.state_dict())
    x = torch.randint(0, 1024, (2, 33))
    loss_a, d_a = CrossEntropyLoss(z_loss=1e-4)(model(x[:, :-1]).logits, x[:, 1:])
    out = fused(x[:, :-1], target=x[:, 1:])
    assert torch.allclose(loss_a, out.loss, atol=1e-5)
    assert torch.allclose(d_a["z-loss"] * 1e-4 if False else out.loss_dict["cross entropy"], d_a["cross entropy"], atol=1e-5)


def test_activation_checkpointing_same_grads(zoo):
    torch.manual_seed(0)
    model = instantiate(tiny_llama_conf(zoo, n_layers=2))
    model.init_weights()
    x = torch.randint(0, 1024, (2, 17))
    model(x).logits.square().mean().backward()
    g0 = [p.grad.clone() for p in model.parameters()]
    model.zero_grad()
    model.gradient_checkpointing_enable(1)
    model.train()
    model(x).logits.square().mean().backward()
    for a, p in zip(g0, model.parameters()):
        assert torch.allclose(a, p.grad, atol=1e-6)


def test_micro_batches_accumulate_in_every_sharding_unit(zoo):
    """Several backward passes before one optimizer step (PPO micro-batches): the flat gradient
    buffers of the block units and of the root unit hold the sum, and the optimizer step starts
    a new sum."""
    from halite_b200.optim import build_optimizer
    from halite_b200.parallel import parallelize

    torch.manual_seed(0)
    model = parallelize(instantiate(tiny_llama_conf(zoo, n_layers=2)), param_dtype="float32",
                        reduce_dtype="float32", device="cpu")
    model.init_weights("cpu")
    opt = build_optimizer(partial(torch.optim.AdamW, lr=0.0), model, weight_decay=0.0)
    a, b = torch.randint(0, 1024, (2, 16)), torch.randint(0, 1024, (2, 16))

    def grads(batches):
        opt.zero_grad()
        for x in batches:
            model(x).logits.float().logsumexp(-1).sum().backward()
        model._hb_fsdp.finish_backward()
        return [u.full_grad.clone() for u in model._hb_fsdp.units]

    ga, gb, gab = grads([a]), grads([b]), grads([a, b])
    for x, y, z in zip(ga, gb, gab):
        torch.testing.assert_close(z, x + y, atol=1e-5, rtol=1e-5)
    opt.step()                                   # consumes the sum (learning rate 0: weights unchanged)
    for x, z in zip(ga, grads([a])):
        torch.testing.assert_close(z, x, atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("config", [{"mode": "full"}, {"mode": "full", "every": 2}, {"mode": "selective", "selective": "2"},
                                    {"mode": "selective", "selective": "op"}])
def test_activation_checkpointing_modes_leave_gradients_unchanged(zoo, config):
    """Full, every-N, every-k-th-block and per-op (feed-forward half) checkpointing recompute
    activations but must produce the gradients of the plain run."""
    from halite_b200.conf import instantiate
    from halite_b200.parallel import parallelize
    from tests.conftest import tiny_llama_conf

    def grads(ac_config):
        torch.manual_seed(0)
        model = instantiate(tiny_llama_conf(zoo, n_layers=4, dim=64, intermediate_size=96, n_heads=2, head_dim=32,
                                            n_key_value_heads=1, vocab_size=128))
        model.init_weights()
        if ac_config is not None:
            model = parallelize(model, None, None, param_dtype="float32", reduce_dtype="float32", device="cpu",
                                activation_checkpointing=True, activation_checkpointing_config=ac_config)
        else:
            model = parallelize(model, None, None, param_dtype="float32", reduce_dtype="float32", device="cpu")
        model.train()
        x = torch.randint(0, 128, (2, 17), generator=torch.Generator().manual_seed(1))
        loss = torch.nn.functional.cross_entropy(model(x[:, :-1]).logits.flatten(0, 1), x[:, 1:].flatten())
        loss.backward()
        model._hb_fsdp.finish_backward()
        return loss.item(), [u.full_grad.clone() for u in model._hb_fsdp.units]

    base_loss, base = grads(None)
    loss, got = grads(config)
    assert abs(loss - base_loss) < 1e-6
    for a, b in zip(base, got):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)

    with pytest.raises(ValueError):
        grads({"mode": "sometimes"})
