"""Checkpoint conversion: native -> Meta-style tensor-parallel shards -> native round trip, the
fused-projection post-processing, the command-line tool, generation with dense caches and the
attention-mask programs."""

import os
import sys
from functools import partial

import torch

from halite_b200.conf import function, instantiate
from halite_b200.conf.loader import load_module
from halite_b200.models.convert import (Policy, convert_checkpoint, convert_state_dict, get_matched_keys)
from tests.helpers import ROOT

zoo = load_module(os.path.join(ROOT, "configs/models/transformer.py"))


class maps_mod:
    """The map builders as an experiment would get them: through `function(...)` references."""

    _m = load_module(os.path.join(ROOT, "configs/models/checkpoint_maps.py"))
    decoder_weight_maps = staticmethod(instantiate(function(_m.decoder_weight_maps)))
    fuse_projections = staticmethod(instantiate(function(_m.fuse_projections)))
    unfuse_projections = staticmethod(instantiate(function(_m.unfuse_projections)))


def tiny(qkv_split=True, **kw):
    cfg = zoo.transformer(vocab_size=128, dim=64, n_heads=4, head_dim=16, n_layers=2, intermediate_size=176,
                          context_len=64, n_key_value_heads=2, rms_norm_epsilon=1e-5, qkv_split=qkv_split,
                          gated_ff_split=qkv_split, init=partial(torch.nn.init.normal_, std=0.2), **kw)
    torch.manual_seed(0)
    m = instantiate(cfg)
    m.init_weights()
    return m.eval()


def test_round_trip_through_two_meta_shards_and_fused_layout():
    model = tiny()
    sd = model.state_dict()
    conf = {"qkv_split": True, "gated_ff_split": True}
    policy = Policy(weight_maps=maps_mod.decoder_weight_maps("meta"), to_halite_postprocess=maps_mod.fuse_projections,
                    from_halite_preprocess=maps_mod.unfuse_projections)
    shards = convert_checkpoint(sd, conf, policy, mode="from_halite", n_shards=2)
    assert len(shards) == 2 and "layers.1.attention.wq.weight" in shards[0]
    assert shards[0]["layers.0.attention.wo.weight"].shape == (64, 32)        # row-parallel: cut on dim 1
    assert shards[0]["layers.0.attention_norm.weight"].shape == (64,)
    # the model names the split gated MLP linear_proj / linear_out; Meta maps know linear1 / linear2
    back = convert_checkpoint(shards, conf, policy, mode="to_halite")
    missing = [k for k in sd if k not in back]
    assert not missing, missing
    assert all(torch.equal(back[k], sd[k]) for k in sd)
    # same shards into a model with fused qkv and fused gate|up
    fused = tiny(qkv_split=False)
    got = convert_checkpoint(shards, {"qkv_split": False, "gated_ff_split": False}, policy, mode="to_halite")
    fused.load_state_dict(got)
    x = torch.randint(0, 128, (2, 9))
    torch.testing.assert_close(fused(x).logits, model(x).logits, rtol=1e-5, atol=1e-5)


def test_hf_names_and_matched_keys():
    maps = maps_mod.decoder_weight_maps("hf", qk_norm=True)
    hf = {"model.layers.3.self_attn.q_norm.weight": torch.ones(4), "model.embed_tokens.weight": torch.ones(2, 2),
          "unrelated.weight": torch.ones(1)}
    out = convert_state_dict(hf, maps)
    assert set(out) == {"blocks.3.self_attention.module.attention.q_norm.weight", "embedding.embed_input_ids.weight"}
    assert set(convert_state_dict(out, maps, reverse=True)) == set(hf) - {"unrelated.weight"}
    keys = [f"blocks.{i}.ff.module.linear1.weight" for i in (10, 2, 1)]
    assert get_matched_keys(keys, "blocks.#.ff.module.linear1.weight")[0].startswith("blocks.1.")


def test_convert_tool_writes_a_loadable_model_folder(tmp_path):
    sys.path.insert(0, os.path.join(ROOT, "scripts/tools"))
    import convert_checkpoint as tool

    from halite_b200.distributed.checkpoint import load_checkpoint

    conf_file = tmp_path / "configs" / "tiny.py"
    conf_file.parent.mkdir()
    conf_file.write_text(f'''
from functools import partial
from torch import nn
from halite_b200.conf import call, field, function
from halite_b200.conf.loader import load_module
_zoo = load_module("{ROOT}/configs/models/transformer.py")
_maps = load_module("{ROOT}/configs/models/checkpoint_maps.py")
conf = field()
_t = field(vocab_size=128, dim=64, n_heads=4, head_dim=16, n_layers=2, intermediate_size=176, context_len=64,
           n_key_value_heads=2, rms_norm_epsilon=1e-5, qkv_split=True, gated_ff_split=True)
conf.model = call[_zoo.transformer](**_t, init=partial(nn.init.normal_, std=0.2))
conf.model_conf = field(**_t)
conf.policy = field(weight_maps=_maps.decoder_weight_maps("meta"), to_halite_postprocess=function(_maps.fuse_projections))
''')
    model = tiny()
    policy = Policy(weight_maps=maps_mod.decoder_weight_maps("meta"),
                    from_halite_preprocess=maps_mod.unfuse_projections)
    shards = convert_checkpoint(model.state_dict(), {}, policy, mode="from_halite", n_shards=2)
    for i, s in enumerate(shards):
        torch.save(s, tmp_path / f"consolidated.{i:02d}.pth")
    out = tmp_path / "out"
    tool.main(["--conf", str(conf_file), "--out", str(out), str(tmp_path / "consolidated.*.pth")])
    assert (out / "config.json").exists() and (out / ".metadata").exists()
    fresh = tiny()
    with torch.no_grad():
        for p in fresh.parameters():
            p.zero_()
    load_checkpoint(fresh, str(out))
    assert all(torch.equal(a, b) for a, b in zip(fresh.parameters(), model.parameters()))


def test_generate_matches_recompute_with_both_cache_kinds():
    from halite_b200.models.cache_manager import AllocatedCacheManager, BasicCacheManager

    model = tiny()
    prompt = torch.randint(0, 128, (3, 5))
    want = prompt.clone()
    for _ in range(6):
        want = torch.cat((want, model(want).logits[:, -1].argmax(-1)[:, None]), 1)
    assert torch.equal(model.generate(prompt, max_new_tokens=6, temperature=0), want)
    mgr = AllocatedCacheManager(2, 3, 32, 2, 16, device="cpu")
    assert torch.equal(model.generate(prompt, max_new_tokens=6, temperature=0, cache=mgr), want)
    assert mgr.lengths == [10, 10]
    assert torch.equal(model.generate(prompt, max_new_tokens=6, temperature=0, cache=BasicCacheManager(2)), want)
    # eos stops a row and pads it afterwards
    eos = int(want[0, 6])
    out = model.generate(prompt, max_new_tokens=6, temperature=0, eos_token_id=eos, pad_token_id=0)
    row = out[0, 5:].tolist()
    assert eos in row and all(t == 0 for t in row[row.index(eos) + 1:])
    # sampling processors keep the distribution inside the top-k set
    g = torch.Generator().manual_seed(0)
    s = model.generate(prompt, max_new_tokens=4, temperature=0.8, top_k=1, generator=g)
    assert torch.equal(s, want[:, :9])


def test_mask_programs():
    from halite_b200.models.flex_attention import (BatchDocumentMask, BidirectionalMask, CausalMask, ComposeMask,
                                                    FlexAttentionProcessor, SlidingWindowCausalMask,
                                                    batch_length_to_offsets)
    from halite_b200.ops.attention import attention_reference

    off = batch_length_to_offsets([[3, 5], [4, 2, 2]])
    r = FlexAttentionProcessor(block_mask=BatchDocumentMask(CausalMask()))(
        batch=2, q_len=8, kv_len=8, device="cpu", document_offsets=off)
    allowed = ~r.dense("cpu")
    assert allowed[0, 0, 2, :3].all() and not allowed[0, 0, 3, :3].any() and allowed[1, 0, 7, 6:].all()
    assert not allowed[1, 0, 6, 4:6].any()
    # packed rows attend like separate sequences
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 8, 2, 16) for _ in range(3))
    packed = attention_reference(q, k, v, causal=False, mask=r.dense("cpu")[:1])
    alone = attention_reference(q[:, 3:], k[:, 3:], v[:, 3:], causal=True)
    torch.testing.assert_close(packed[:, 3:], alone, rtol=1e-5, atol=1e-5)
    sw = FlexAttentionProcessor(block_mask=SlidingWindowCausalMask(2))(batch=1, q_len=6, kv_len=6, device="cpu")
    assert sw.to_attention_kwargs(6, 6, "cpu") == {"causal": True, "window": 2}
    bid = torch.tensor([[0, 1, 1, 1, 0, 0]])
    b = FlexAttentionProcessor(block_mask=BidirectionalMask(CausalMask()))(
        batch=1, q_len=6, kv_len=6, device="cpu", bidirection_ids=bid)
    a = ~b.dense("cpu")[0, 0]
    assert a[1, 3] and not a[0, 1] and a[5, 0] and not a[4, 5]
    comp = ComposeMask(CausalMask(), SlidingWindowCausalMask(1))
    assert comp.inputs == ()
    m = comp()
    i = torch.arange(4)
    assert m(0, 0, i[:, None], i[None, :]).int().sum() == 7
