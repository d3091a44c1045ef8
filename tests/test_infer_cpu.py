"""Paged-KV engine on CPU (tiny Llama, page size 16, 8 prompts of 16 tokens): greedy decode through
the paged cache must reproduce the dense forward (tokens equal, log-probs within 1e-4), the
prefix cache must be hit by shared prefixes, and no page or request slot may leak."""

from functools import partial

import pytest
import torch

from halite_b200.conf import instantiate
from halite_b200.infer import InferenceEngine, InferenceRequest, ModelConfig, ServerConfig
from halite_b200.infer.memory_pool import PagedKVPool, RequestToPagePool
from halite_b200.infer.radix_cache import RadixCache

KW = dict(vocab_size=1024, dim=256, n_heads=4, head_dim=64, n_layers=4, intermediate_size=688,
          context_len=512, n_key_value_heads=2, rms_norm_epsilon=1e-5, qkv_split=True, gated_ff_split=True)


def build(zoo, server=None, **over):
    kw = dict(KW, init=partial(torch.nn.init.normal_, std=0.02))
    kw.update(over)
    cfg = zoo.transformer(**kw)
    torch.manual_seed(0)
    model = instantiate(cfg)
    model.init_weights()
    model.eval()
    to_infer = instantiate(zoo.transformer_infer(**kw, infer="paged"))
    with torch.device("meta"):
        imodel = instantiate(to_infer(cfg))
    mc = ModelConfig(n_heads=kw["n_heads"], n_key_value_heads=kw["n_key_value_heads"], head_dim=kw["head_dim"],
                     n_layers=kw["n_layers"], context_len=kw["context_len"], device="cpu",
                     kv_cache_dtype=torch.float32)
    eng = InferenceEngine(imodel, None, mc, server or ServerConfig(max_total_tokens=4096))
    eng.load_state_dict(model.state_dict())
    return model, eng


def dense_check(model, result, sample=0):
    n_in = len(result.input_ids)
    seq = torch.tensor([result.input_ids + result.output_ids[sample]])
    with torch.no_grad():
        logits = model(seq).logits[0].float()
    lp = torch.log_softmax(logits, -1)[n_in - 1:-1]
    out = torch.tensor(result.output_ids[sample])
    return lp.argmax(-1).tolist(), lp.gather(-1, out[:, None]).squeeze(-1)


@pytest.mark.parametrize("steps_ahead", [1, 4])
def test_paged_greedy_decode_matches_dense(zoo, steps_ahead):
    model, eng = build(zoo, ServerConfig(max_total_tokens=4096, decode_steps_ahead=steps_ahead))
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, 1024, (8, 16), generator=g).tolist()
    res = eng.infer_batch([InferenceRequest(i, p, {"max_new_tokens": 32, "top_k": 1})
                           for i, p in enumerate(prompts)])
    assert len(res) == 8
    for r in res:
        want, lp = dense_check(model, r)
        assert want == r.output_ids[0]
        assert (lp - torch.tensor(r.output_logprobs[0])).abs().max() < 1e-4
        assert r.finish_reason == ["length"]
    sch = eng.scheduler
    assert sch.kv_pool.available_pages() + sch.tree_cache.evictable_pages == sch.kv_pool.num_pages
    assert sch.req_pool.available_size() == eng.model_runner.max_requests
    sch.tree_cache.sanity_check()


def test_prefix_cache_hit_and_n_samples(zoo):
    model, eng = build(zoo)
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, 1024, (40,), generator=g).tolist()
    reqs = [InferenceRequest(i, shared + torch.randint(0, 1024, (5 + i,), generator=g).tolist(),
                             {"max_new_tokens": 6, "top_k": 1}) for i in range(4)]
    first = eng.infer_batch(reqs[:1])
    rest = eng.infer_batch(reqs[1:])
    assert first[0].num_cached_prompt_tokens == [0]
    assert all(r.num_cached_prompt_tokens == [32] for r in rest)      # 2 full pages of the prefix
    for r in first + rest:
        want, _ = dense_check(model, r)
        assert want == r.output_ids[0]
    # n > 1: the prompt is prefilled once, the samples share its pages
    res = eng.infer_batch([InferenceRequest("a", shared, {"max_new_tokens": 5, "n": 3, "temperature": 1.0})])
    assert len(res) == 1 and len(res[0].output_ids) == 3
    assert all(c == 32 for c in res[0].num_cached_prompt_tokens)
    for s in range(3):
        _, lp = dense_check(model, res[0], s)
        assert (lp - torch.tensor(res[0].output_logprobs[s])).abs().max() < 1e-4
    eng.scheduler.tree_cache.sanity_check()


def test_chunked_prefill_and_retraction(zoo):
    # tiny pool: forces eviction, chunked prefill (chunk 32) and decode-time retraction
    server = ServerConfig(max_total_tokens=448, chunked_prefill_size=32, max_prefill_tokens=64,
                          decode_steps_ahead=2, schedule_conservativeness=0.02)
    model, eng = build(zoo, server)
    g = torch.Generator().manual_seed(2)
    reqs = [InferenceRequest(i, torch.randint(0, 1024, (50 + 7 * i,), generator=g).tolist(),
                             {"max_new_tokens": 40, "top_k": 1}) for i in range(6)]
    res = eng.infer_batch(reqs)
    assert len(res) == 6
    for r in res:
        want, lp = dense_check(model, r)
        assert want == r.output_ids[0]
        assert (lp - torch.tensor(r.output_logprobs[0])).abs().max() < 1e-4
    sch = eng.scheduler
    assert sch.kv_pool.available_pages() + sch.tree_cache.evictable_pages == sch.kv_pool.num_pages
    assert sch.req_pool.available_size() == eng.model_runner.max_requests
    assert sch.stats["retractions"] > 0
    sch.tree_cache.sanity_check()


def test_stop_token_and_lifecycle(zoo):
    model, eng = build(zoo)
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, 1024, (20,), generator=g).tolist()
    base = eng.infer_batch([InferenceRequest(0, prompt, {"max_new_tokens": 12, "top_k": 1})])[0]
    stop = base.output_ids[0][5]
    first = base.output_ids[0].index(stop)
    cut = eng.infer_batch([InferenceRequest(1, prompt, {"max_new_tokens": 12, "top_k": 1,
                                                        "stop_token_ids": [stop]})])[0]
    assert cut.output_ids[0] == base.output_ids[0][: first + 1] and cut.finish_reason == ["stop"]
    # hand the memory back and take it again, with the same weights reloaded
    import weakref

    sd = model.state_dict()
    pool = weakref.ref(eng.model_runner.kv_pool)
    eng.cleanup()
    assert eng.model_runner.kv_pool is None
    assert pool() is None                     # scheduler and attention layers let go of it too
    eng.initialize()
    eng.load_state_dict(sd)
    again = eng.infer_batch([InferenceRequest(2, prompt, {"max_new_tokens": 12, "top_k": 1})])[0]
    assert again.output_ids == base.output_ids


def test_resident_engine_takes_new_weights_in_place(zoo):
    """`keep_resident`: cleanup() leaves weights and pools where they are, load_state_dict() copies
    new values into the same storage, and the next rollout follows the new weights."""
    model, eng = build(zoo, ServerConfig(max_total_tokens=4096, keep_resident=True))
    prompts = torch.randint(0, 1024, (4, 12), generator=torch.Generator().manual_seed(1)).tolist()
    reqs = lambda: [InferenceRequest(i, p, {"max_new_tokens": 8, "top_k": 1}) for i, p in enumerate(prompts)]
    first = eng.infer_batch(reqs())
    pool, weight = eng.model_runner.kv_pool, next(eng.model_runner.model.parameters())
    ptr = weight.data_ptr()
    eng.cleanup()
    assert eng.model_runner.kv_pool is pool and not weight.is_meta
    with torch.no_grad():
        for p in model.parameters():
            p.add_(0.05 * torch.randn_like(p))
    eng.initialize()
    eng.load_state_dict(model.state_dict())
    assert next(eng.model_runner.model.parameters()).data_ptr() == ptr
    assert eng.model_runner.kv_pool.available_pages() == pool.num_pages if hasattr(pool, "num_pages") else True
    second = eng.infer_batch(reqs())
    for r in second:
        want, lp = dense_check(model, r)
        assert want == r.output_ids[0]
        assert (lp - torch.tensor(r.output_logprobs[0])).abs().max() < 1e-4
    assert any(a.output_ids != b.output_ids for a, b in zip(first, second))


def test_sampler_distribution_and_filters():
    from halite_b200.infer.batch import BatchSamplingParams
    from halite_b200.infer.sampler import Sampler
    from halite_b200.infer.types import SamplingParams

    class R:
        def __init__(self, **kw):
            self.sampling_params = SamplingParams(**kw)

    torch.manual_seed(0)
    logits = torch.tensor([[2.0, 1.0, 0.5, -1.0, -3.0]]).repeat(20000, 1)
    s = Sampler()
    g = torch.Generator().manual_seed(0)
    sp = BatchSamplingParams.from_requests([R(temperature=1.0)] * 20000, "cpu")
    ids, lp = s(logits, sp, g)
    freq = torch.bincount(ids, minlength=5).float() / 20000
    assert (freq - torch.softmax(logits[0], -1)).abs().max() < 0.015
    assert torch.allclose(lp, torch.log_softmax(logits, -1).gather(-1, ids[:, None]).squeeze(-1), atol=1e-6)
    sp = BatchSamplingParams.from_requests([R(temperature=1.0, top_k=2)] * 20000, "cpu")
    ids, _ = s(logits, sp, g)
    assert set(ids.tolist()) == {0, 1}
    sp = BatchSamplingParams.from_requests([R(temperature=1.0, top_p=0.7)] * 20000, "cpu")
    ids, _ = s(logits, sp, g)
    assert set(ids.tolist()) == {0, 1}          # p0 = 0.61 < 0.7, so the second token is kept too
    sp = BatchSamplingParams.from_requests([R(temperature=1.0, min_p=0.5)] * 20000, "cpu")
    ids, _ = s(logits, sp, g)
    assert set(ids.tolist()) == {0}             # p1 / p0 = 0.37 < 0.5
    sp = BatchSamplingParams.from_requests([R(temperature=0.0)] * 4, "cpu")
    ids, _ = s(logits[:4], sp, g)
    assert ids.tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("backend", ["python", "native"])
def test_radix_cache_pages(backend):
    from halite_b200.infer.radix_cache import make_radix_cache

    pool = PagedKVPool(64, 4, 1, 1, 8, torch.float32, "cpu")
    tree = make_radix_cache(4, pool, backend=backend)
    a = list(range(12))
    pa = pool.alloc(3)
    assert tree.insert(a, pa) == 0
    pages, node = tree.match_prefix(a + [99])
    assert pages == pa
    # shares 2 pages, diverges inside the third: the node is split on the page boundary
    b = a[:8] + [50, 51, 52, 53]
    pages_b, node_b = tree.match_prefix(b)
    assert pages_b == pa[:2]
    pb = pool.alloc(1)
    assert tree.insert(b, pa[:2] + pb) == 2
    tree.sanity_check()
    assert tree.evictable_pages == 4
    tree.inc_lock_ref(node_b)
    assert tree.evictable_pages == 2 and tree.protected_pages == 2
    freed = tree.evict(10)
    assert freed == 2 and pool.available_pages() == 64 - 2
    tree.dec_lock_ref(node_b)
    assert tree.evict(10) == 2 and pool.available_pages() == 64
    tree.sanity_check()
    # partial page never matches
    assert tree.match_prefix([1, 2, 3])[0] == []


def test_native_radix_tree_agrees_with_python_under_random_traffic():
    """Random inserts / matches / locks / evictions against both trees: same matched pages,
    same counters, invariants hold; plus the native page allocator."""
    import random

    from halite_b200.infer.radix_cache import NativeRadixCache

    rng = random.Random(0)
    ps = 4
    pools = [PagedKVPool(4096, ps, 1, 1, 8, torch.float32, "cpu") for _ in range(2)]
    trees = [RadixCache(ps, pools[0]), NativeRadixCache(ps, pools[1])]
    stems = [[rng.randrange(50) for _ in range(ps * rng.randrange(1, 6))] for _ in range(8)]
    locked = []
    for step in range(400):
        seq = list(rng.choice(stems)) + [rng.randrange(50) for _ in range(ps * rng.randrange(0, 4))]
        op = rng.random()
        if op < 0.5:
            outs = []
            for tree, pool in zip(trees, pools):
                matched, _ = tree.match_prefix(seq)
                fresh = pool.alloc(len(seq) // ps - len(matched))
                shared = tree.insert(seq[: (len(seq) // ps) * ps], matched + fresh)
                pool.free(fresh[: max(0, shared - len(matched))])
                outs.append((len(matched), shared))
            assert outs[0] == outs[1]
        elif op < 0.7:
            res = [tree.match_prefix(seq + [7]) for tree in trees]
            assert len(res[0][0]) == len(res[1][0])
            if res[0][0] and len(locked) < 6:
                for tree, (_, node) in zip(trees, res):
                    tree.inc_lock_ref(node)
                locked.append([r[1] for r in res])
        elif op < 0.8 and locked:
            nodes = locked.pop(rng.randrange(len(locked)))
            for tree, node in zip(trees, nodes):
                tree.dec_lock_ref(node)
        else:
            n = rng.randrange(1, 12)
            assert trees[0].evict(n) == trees[1].evict(n)
        assert trees[0].evictable_pages == trees[1].evictable_pages
        assert trees[0].protected_pages == trees[1].protected_pages
        assert pools[0].available_pages() == pools[1].available_pages()
        if step % 50 == 0:
            for tree in trees:
                tree.sanity_check()
    assert trees[0].total_pages() == trees[1].total_pages() > 0
    alloc = trees[1]._ext.PageAllocator(10)
    first = alloc.alloc(3)
    assert first == [3, 2, 1] or sorted(first) == [1, 2, 3]
    assert alloc.alloc(8) is None and alloc.available() == 7
    alloc.free(first)
    assert alloc.available() == 10 and alloc.capacity() == 10


def test_tensor_parallel_engine_matches_dense_on_two_ranks():
    """tp=2 over Gloo: each rank holds its slice of the projections and its KV heads, the ranks
    take identical scheduling and sampling decisions, and the tokens equal dense decoding."""
    import os

    from tests.helpers import ROOT, run_ranks

    outs = run_ranks(os.path.join(ROOT, "tests/ranks/infer_tp.py"), 2, timeout=600)
    assert all(o.count("TP_OK") == 2 for o in outs), outs[0][-3000:]


def test_decode_graphs_are_only_captured_when_attention_runs_the_paged_kernels(zoo):
    """The plain-PyTorch attention path reads lengths on the host, which a stream capture forbids: the
    runner must decide from the model whether a decode forward is capturable."""
    _, eng = build(zoo)
    runner = eng.model_runner
    assert runner._graph_for(4) is None                      # CPU: never
    assert runner._graph_capturable() is False               # fp32 cache and weights here
    runner._capturable = None
    runner.kv_cache_dtype = torch.bfloat16
    for p in runner.model.parameters():
        p.data = p.data.to(torch.bfloat16)
    assert runner._graph_capturable() is True                # head_dim 64, bf16 everywhere
    runner._capturable = None
    runner.model_config.head_dim = 16
    assert runner._graph_capturable() is False               # a head size the kernels do not cover
    runner.model_config.head_dim = 64
    runner._capturable = None
    attn = next(m for m in runner.model.modules() if hasattr(m, "softcap"))
    attn.softcap = 30.0
    assert runner._graph_capturable() is False               # soft-capped scores run the PyTorch path
