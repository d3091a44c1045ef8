"""sm_100a inference kernels against the gather-and-dense reference, and the engine end to end
on the GPU (eager and CUDA-graph decode)."""

import math
from functools import partial

import pytest
import torch

pytestmark = pytest.mark.gpu


def make_cache(n_req, seq_lens, hk, d, page_size=16, extra_pages=7, seed=0):
    from halite_b200.infer.batch import ForwardBatch, ForwardMode

    g = torch.Generator(device="cuda").manual_seed(seed)
    n_pages = sum((s + page_size - 1) // page_size for s in seq_lens) + extra_pages
    k_cache = torch.randn(n_pages + 1, page_size, hk, d, device="cuda", generator=g).bfloat16()
    v_cache = torch.randn(n_pages + 1, page_size, hk, d, device="cuda", generator=g).bfloat16()
    perm = (torch.randperm(n_pages, device="cuda", generator=g) + 1).int()
    max_pages = max((s + page_size - 1) // page_size for s in seq_lens) + 2
    table = torch.zeros(n_req + 3, max_pages, dtype=torch.int32, device="cuda")
    slots = torch.arange(n_req, device="cuda").flip(0).int() + 1   # non-trivial slot order
    used = 0
    for i, s in enumerate(seq_lens):
        n = (s + page_size - 1) // page_size
        table[slots[i], :n] = perm[used:used + n]
        used += n
    return k_cache, v_cache, table, slots.contiguous()


@pytest.mark.parametrize("hq,hk,d", [(24, 8, 128), (32, 8, 128), (8, 8, 128), (16, 2, 64), (4, 2, 64)])
@pytest.mark.parametrize("batch", [1, 7, 150])
def test_paged_decode(hq, hk, d, batch):
    from halite_b200.infer.batch import ForwardBatch, ForwardMode
    from halite_b200.ops import paged_attention as pa

    torch.manual_seed(batch)
    seq_lens = [1, 15, 16, 17, 63, 64, 65, 700, 1033][:batch] if batch < 10 else \
        torch.randint(1, 900, (batch,)).tolist()
    seq_lens = (seq_lens * ((batch + len(seq_lens) - 1) // len(seq_lens)))[:batch]
    k_cache, v_cache, table, slots = make_cache(batch, seq_lens, hk, d)
    q = torch.randn(batch, hq, d, device="cuda").bfloat16()
    fb = ForwardBatch(mode=ForwardMode.DECODE, input_ids=None, positions=None, out_cache_loc=None,
                      req_slots=slots, seq_lens=torch.tensor(seq_lens, dtype=torch.int32, device="cuda"),
                      page_table=table, max_seq_len=max(seq_lens), seq_lens_cpu=seq_lens)
    ws = torch.empty(batch * hq * 32 * (d + 2), dtype=torch.float32, device="cuda")
    out = pa.paged_decode_attention(q, k_cache, v_cache, fb, workspace=ws)
    ref = pa.paged_attention_reference(q.float(), k_cache.float(), v_cache.float(), fb)
    assert (out.float() - ref).abs().max() < 2e-2
    out1 = pa.paged_decode_attention(q, k_cache, v_cache, fb, workspace=None)   # single split
    assert (out1.float() - ref).abs().max() < 2e-2


@pytest.mark.parametrize("hq,hk,d", [(24, 8, 128), (8, 2, 64)])
def test_paged_prefill_with_prefix(hq, hk, d):
    from halite_b200.infer.batch import ForwardBatch, ForwardMode
    from halite_b200.ops import paged_attention as pa

    torch.manual_seed(0)
    prefix = [0, 16, 48, 0, 128, 32]
    extend = [1, 5, 64, 130, 257, 63]
    seq_lens = [p + e for p, e in zip(prefix, extend)]
    B = len(seq_lens)
    k_cache, v_cache, table, slots = make_cache(B, seq_lens, hk, d)
    T = sum(extend)
    wide = torch.randn(T, (hq + 2 * hk) * d, device="cuda").bfloat16()
    q = wide[:, : hq * d].unflatten(-1, (hq, d))       # strided rows, like a packed qkv output
    indptr = [0]
    for e in extend:
        indptr.append(indptr[-1] + e)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    fb = ForwardBatch(mode=ForwardMode.EXTEND, input_ids=None, positions=None, out_cache_loc=None,
                      req_slots=slots, seq_lens=i32(seq_lens), extend_lens=i32(extend),
                      prefix_lens=i32(prefix), qo_indptr=i32(indptr), page_table=table,
                      max_seq_len=max(seq_lens), max_extend_len=max(extend), seq_lens_cpu=seq_lens,
                      extend_lens_cpu=extend)
    out = pa.paged_prefill_attention(q, k_cache, v_cache, fb)
    ref = pa.paged_attention_reference(q.float(), k_cache.float(), v_cache.float(), fb)
    assert (out.float() - ref).abs().max() < 3e-2


@pytest.mark.parametrize("interleaved", [True, False])
def test_rope_append(interleaved):
    from halite_b200 import ops
    from halite_b200.models.position import RotaryTable
    from halite_b200.ops import paged_attention as pa
    from halite_b200.ops.rope import apply_rope_reference, rope_tables

    torch.manual_seed(1)
    T, hq, hk, d = 77, 24, 8, 128
    inv = 1.0 / (500000 ** (torch.arange(0, d, 2).float() / d))
    cos, sin = rope_tables(inv, 2048, "cuda")
    pos = torch.randint(0, 2048, (T,), device="cuda")
    wide = torch.randn(T, (hq + 2 * hk) * d, device="cuda").bfloat16()
    q = wide[:, : hq * d].unflatten(-1, (hq, d))
    k = wide[:, hq * d:(hq + hk) * d].unflatten(-1, (hk, d))
    v = wide[:, (hq + hk) * d:].unflatten(-1, (hk, d))
    q_ref = apply_rope_reference(q.float(), cos, sin, pos, interleaved)
    k_ref = apply_rope_reference(k.float(), cos, sin, pos, interleaved)
    v_ref = v.clone()
    k_cache = torch.zeros(20, 16, hk, d, device="cuda", dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    loc = torch.randperm(19 * 16, device="cuda")[:T] + 16
    q_out = pa.rope_append(q, k, v, k_cache, v_cache, RotaryTable(cos, sin, pos, interleaved), loc)
    assert (q_out.float() - q_ref).abs().max() < 2e-2
    assert (k_cache.view(-1, hk, d)[loc].float() - k_ref).abs().max() < 2e-2
    assert torch.equal(v_cache.view(-1, hk, d)[loc], v_ref)
    untouched = torch.ones(20 * 16, dtype=torch.bool, device="cuda")
    untouched[loc] = False
    assert k_cache.view(-1, hk, d)[untouched].abs().max() == 0


def test_sample_gumbel_kernel():
    from halite_b200 import ops

    C = ops.ext()
    torch.manual_seed(2)
    V = 1000
    base = torch.randn(V, device="cuda") * 2
    logits = base.repeat(8192, 1).contiguous()
    temps = torch.full((8192,), 0.8, device="cuda")
    greedy = torch.zeros(8192, dtype=torch.bool, device="cuda")
    ids, lp = C.sample_gumbel(logits, temps, greedy, 0, 1)
    p = torch.softmax(base / 0.8, -1)
    freq = torch.bincount(ids, minlength=V).float() / 8192
    top = p.topk(5).indices
    assert (freq[top] - p[top]).abs().max() < 0.02
    want_lp = torch.log_softmax(logits / 0.8, -1).gather(-1, ids[:, None]).squeeze(-1)
    assert torch.allclose(lp, want_lp, atol=1e-3)
    ids2, _ = C.sample_gumbel(logits, temps, greedy, 0, 2)
    assert (ids != ids2).any()
    greedy[:] = True
    ids3, lp3 = C.sample_gumbel(logits, temps, greedy, 0, 3)
    assert (ids3 == base.argmax()).all()
    big = torch.randn(4, 128256, device="cuda")
    ids4, lp4 = C.sample_gumbel(big, torch.ones(4, device="cuda"), torch.ones(4, dtype=torch.bool, device="cuda"), 1, 1)
    assert torch.equal(ids4, big.argmax(-1))
    assert torch.allclose(lp4, torch.log_softmax(big, -1).max(-1).values, atol=1e-3)


@pytest.mark.parametrize("cudagraph", [False, True])
def test_engine_gpu_matches_dense(zoo, cudagraph):
    from halite_b200.conf import instantiate
    from halite_b200.infer import InferenceEngine, InferenceRequest, ModelConfig, ServerConfig

    kw = dict(vocab_size=2048, dim=512, n_heads=8, head_dim=64, n_layers=3, intermediate_size=1024,
              context_len=512, n_key_value_heads=2, rms_norm_epsilon=1e-5, qkv_split=True,
              gated_ff_split=True, init=partial(torch.nn.init.normal_, std=0.05))
    cfg = zoo.transformer(**kw)
    torch.manual_seed(0)
    model = instantiate(cfg)
    model.init_weights()
    model = model.cuda().bfloat16().eval()
    to_infer = instantiate(zoo.transformer_infer(**kw, infer="paged"))
    with torch.device("meta"):
        imodel = instantiate(to_infer(cfg))
    mc = ModelConfig(n_heads=8, n_key_value_heads=2, head_dim=64, n_layers=3, context_len=512, device="cuda")
    sc = ServerConfig(max_total_tokens=16384, decode_steps_ahead=4, use_cudagraph=cudagraph,
                      cudagraph_step=8, cudagraph_max_batch_size=32)
    eng = InferenceEngine(imodel, None, mc, sc)
    eng.load_state_dict(model.state_dict())
    g = torch.Generator().manual_seed(3)
    shared = torch.randint(0, 2048, (48,), generator=g).tolist()
    reqs = []
    for i in range(12):
        own = torch.randint(0, 2048, (5 + 9 * i,), generator=g).tolist()
        reqs.append(InferenceRequest(i, (shared if i % 2 else []) + own, {"max_new_tokens": 24, "top_k": 1}))
    res = eng.infer_batch(reqs[:2])          # seeds the prefix cache with the shared prompt
    res += eng.infer_batch(reqs[2:])
    assert len(res) == 12
    from halite_b200 import ops

    ops.check_status()
    agree = total = 0
    for r in res:
        n_in = len(r.input_ids)
        seq = torch.tensor([r.input_ids + r.output_ids[0]], device="cuda")
        with torch.no_grad():
            logits = model(seq).logits[0].float()
        lp = torch.log_softmax(logits, -1)[n_in - 1:-1]
        out = torch.tensor(r.output_ids[0], device="cuda")
        got = torch.tensor(r.output_logprobs[0], device="cuda")
        want = lp.gather(-1, out[:, None]).squeeze(-1)
        assert (want - got).abs().max() < 0.15, (want - got).abs().max()
        agree += (lp.argmax(-1) == out).sum().item()
        total += out.numel()
    assert agree / total > 0.9
    sch = eng.scheduler
    assert sch.kv_pool.available_pages() + sch.tree_cache.evictable_pages == sch.kv_pool.num_pages
    assert sch.stats["cached_tokens"] > 0


def test_tokainfer_engine_gpu_matches_dense(zoo):
    """Engine B on the device: mixed prefill + decode forwards scheduled ahead; generated tokens'
    log-probs must agree with a dense bf16 evaluation of the same sequences."""
    from halite_b200.conf import instantiate
    from halite_b200.infer import InferenceRequest, ModelConfig
    from halite_b200.tokainfer import InferenceEngine, ServerConfig

    kw = dict(vocab_size=2048, dim=512, n_heads=8, head_dim=64, n_layers=3, intermediate_size=1024,
              context_len=512, n_key_value_heads=2, rms_norm_epsilon=1e-5, qkv_split=True,
              gated_ff_split=True, init=partial(torch.nn.init.normal_, std=0.05))
    cfg = zoo.transformer(**kw)
    torch.manual_seed(0)
    model = instantiate(cfg)
    model.init_weights()
    model = model.cuda().bfloat16().eval()
    with torch.device("meta"):
        imodel = instantiate(instantiate(zoo.transformer_infer(**kw, infer="paged"))(cfg))
    mc = ModelConfig(n_heads=8, n_key_value_heads=2, head_dim=64, n_layers=3, context_len=512, device="cuda")
    eng = InferenceEngine(imodel, None, mc, ServerConfig(kv_cache_num_tokens=16384, scheduling_steps_ahead=4,
                                                         max_tokens_per_forward=256))
    eng.load_state_dict(model.state_dict())
    g = torch.Generator().manual_seed(3)
    shared = torch.randint(0, 2048, (48,), generator=g).tolist()
    reqs = [InferenceRequest(i, (shared if i % 2 else []) + torch.randint(0, 2048, (5 + 9 * i,), generator=g).tolist(),
                             {"max_new_tokens": 24, "top_k": 1}) for i in range(12)]
    res = eng.infer_batch(reqs)
    from halite_b200 import ops

    ops.check_status()
    worst = 0.0
    for r in res:
        n_in = len(r.input_ids)
        seq = torch.tensor([r.input_ids + r.output_ids[0]], device="cuda")
        with torch.no_grad():
            lp = torch.log_softmax(model(seq).logits[0].float(), -1)[n_in - 1:-1]
        out = torch.tensor(r.output_ids[0], device="cuda")
        got = torch.tensor(r.output_logprobs[0], device="cuda")
        worst = max(worst, (lp.gather(-1, out[:, None]).squeeze(-1) - got).abs().max().item())
        assert len(r.output_ids[0]) == 24
    assert worst < 0.15, worst
    eng.manager.allocator.sanity_checks(set())


def test_page_id_outside_the_pool_raises_the_status_word():
    """A corrupted page table entry is not silently served from page 0: the kernel still reads
    in bounds, and the status word makes the next `check_status()` raise."""
    import halite_b200.ops as ops

    C = ops.ext()
    ops.check_status()
    pages, hk, hq, D = 8, 2, 4, 128
    k_cache = torch.randn(pages, 16, hk, D, device="cuda").bfloat16()
    v_cache = torch.randn(pages, 16, hk, D, device="cuda").bfloat16()
    q = torch.randn(1, hq, D, device="cuda").bfloat16()
    out = torch.empty_like(q)
    table = torch.tensor([[1, 99, 3, 0]], dtype=torch.int32, device="cuda")       # 99: no such page
    slots = torch.zeros(1, dtype=torch.int32, device="cuda")
    lens = torch.tensor([40], dtype=torch.int32, device="cuda")
    C.paged_decode(q, k_cache, v_cache, out, table, slots, lens, None, 0.1, ops.status_word("cuda"))
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="page id"):
        ops.check_status()
    ops.check_status()          # cleared by the report
    assert torch.isfinite(out.float()).all()
