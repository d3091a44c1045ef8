"""Engine B on CPU: block allocator with prefix tree, scheduling arithmetic, completion-length
predictor, shared-prefix grouping, and the manager + worker engine against dense greedy decoding
(schedule-ahead, chunked prefill, prefix reuse, bumping under memory pressure, worker process)."""

import math
import os
from functools import partial

import pytest
import torch

from halite_b200.conf import instantiate
from halite_b200.conf.loader import load_module
from halite_b200.infer.types import InferenceRequest, ModelConfig
from halite_b200.tokainfer import InferenceEngine, ServerConfig
from halite_b200.tokainfer.allocator import BatchIndexAllocator, BlockAllocator, NoSpaceException
from halite_b200.tokainfer.hydragen import group_for_hydragen, reorder_decoding_seqs_for_hydragen
from halite_b200.tokainfer.scheduler import (calc_block_usage_over_time, calc_prefill_per_forward, simulate_blocks,
                                             try_onboarding_seqs)
from halite_b200.tokainfer.stopping_predictor import EarlyStoppingTracker, calc_cumulative_mean_stds
from halite_b200.tokainfer.types import SamplingParams, Sequence
from tests.helpers import ROOT

KW = dict(vocab_size=512, dim=128, n_heads=4, head_dim=32, n_layers=2, intermediate_size=344, context_len=256,
          n_key_value_heads=2, rms_norm_epsilon=1e-5, qkv_split=True, gated_ff_split=True)


def build_pair():
    zoo = load_module(os.path.join(ROOT, "configs/models/transformer.py"))
    kw = dict(KW, init=partial(torch.nn.init.normal_, std=0.05))
    cfg = zoo.transformer(**kw)
    torch.manual_seed(0)
    model = instantiate(cfg)
    model.init_weights()
    model.eval()
    with torch.device("meta"):
        imodel = instantiate(instantiate(zoo.transformer_infer(**kw, infer="paged"))(cfg))
    return model, imodel


def model_config():
    return ModelConfig(n_heads=4, n_key_value_heads=2, head_dim=32, n_layers=2, context_len=256, device="cpu",
                       kv_cache_dtype=torch.float32)


def build_infer_model_for_worker():
    """Picklable factory used by the worker process (weights arrive later by load_state_dict)."""
    _, imodel = build_pair()
    return imodel


def dense_greedy(model, prompt, n):
    ids = torch.tensor([prompt])
    with torch.no_grad():
        for _ in range(n):
            ids = torch.cat((ids, model(ids).logits[:, -1].argmax(-1)[:, None]), 1)
    return ids[0, len(prompt):].tolist()


def test_block_allocator_prefix_tree():
    a = BlockAllocator(16, 4)
    prompt = list(range(10))                       # 2 full pages + 2 tokens
    cached, fresh = a.allocate_with_prefix_match("s1", prompt)
    assert cached == [] and len(fresh) == 3 and a.num_free_blocks() == 13
    grown = a.allocate_up_to_length("s1", fresh, 13)
    assert len(grown) == 1
    a.free_and_update("s1", fresh + grown, prompt + [90, 91, 92])           # 13 tokens -> 3 full pages cached
    a.sanity_checks(set())
    assert a.num_free_blocks() == 16                                        # cached pages are reclaimable
    # same prompt again: the first two pages are reused, never the page of the last prompt token
    cached2, fresh2 = a.allocate_with_prefix_match("s2", prompt)
    assert cached2 == fresh[:2] and len(fresh2) == 1
    # a 12-token prompt (exactly 3 pages) may reuse only 2: its last token must be computed
    cached3, fresh3 = a.allocate_with_prefix_match("s3", prompt + [90, 91])
    assert cached3 == fresh[:2] and len(fresh3) == 1
    a.sanity_checks({"s2", "s3"})
    with pytest.raises(NoSpaceException):
        a.allocate_with_prefix_match("big", list(range(100, 200)))
    a.sanity_checks({"s2", "s3"})                                            # failed allocation leaves nothing behind
    a.free_and_update("s2", cached2 + fresh2, prompt)
    a.free_and_update("s3", cached3 + fresh3, prompt + [90, 91])
    a.sanity_checks(set())
    # filling the pool evicts unused tree leaves, least recently used first
    got = a.allocate_up_to_length("fill", [], 16 * 4)
    assert len(got) == 16 and a.num_free_blocks() == 0 and a.prefix_match(prompt) == []
    idx = BatchIndexAllocator(2)
    r0, r1 = idx.allocate(), idx.allocate()
    with pytest.raises(NoSpaceException):
        idx.allocate()
    idx.free_index(r0)
    assert idx.allocate() == r0 and r1 != r0


def _seq(prompt_len, scheduled_prompt=None, decode=0, max_new=64, kv=None, sid=None):
    s = Sequence(sid or f"s{prompt_len}-{decode}", 0, list(range(prompt_len)), SamplingParams(max_new_tokens=max_new))
    s.prompt_scheduled = prompt_len if scheduled_prompt is None else scheduled_prompt
    s.decode_scheduled = decode
    s.kv_indices = kv or []
    return s


def test_scheduling_arithmetic():
    ps = 16
    # one sequence: 40 prompt tokens (3 pages), 30 more tokens -> 70 tokens = 5 pages, then freed
    u = calc_block_usage_over_time([_seq(40)], ps, [30])
    assert u.points[0].blocks == 3 and u.peak == 5 and u.points[-1].blocks == 0
    steps = {p.step: p.blocks for p in u.points}
    assert steps[9] == 4 and steps[25] == 5                 # lengths 49 and 65 open pages
    # two sequences finishing at different times never overlap their peaks beyond the sum
    u2 = calc_block_usage_over_time([_seq(40), _seq(16, decode=0)], ps, [30, 100])
    assert u2.peak == max(p.blocks for p in u2.points) <= 5 + math.ceil(116 / 16)
    assert simulate_blocks([0] * 15 + [4], 1) == 0 and simulate_blocks([3] + [0] * 15, 1) == 3
    assert simulate_blocks([0, 2] + [0] * 14, 16) == 2
    running = [_seq(64, decode=10)]
    waiting = [_seq(32, scheduled_prompt=0, sid=f"w{i}") for i in range(10)]
    predict = lambda s: 32
    # each waiting sequence peaks at 4 pages, the running one at ceil((64+32)/16) = 6
    assert try_onboarding_seqs(running, waiting, ps, 6 + 4 * 3, predict) == 3
    assert try_onboarding_seqs(running, waiting, ps, 1000, predict) == 10
    assert try_onboarding_seqs(running, waiting, ps, 7, predict) == 0
    a, b = _seq(100, scheduled_prompt=0, sid="a"), _seq(50, scheduled_prompt=20, sid="b")
    plan = calc_prefill_per_forward([a, b], n_decoding=8, max_tokens_per_forward=96, round_up_multiple=16)
    # 88-token budget: a's chunk is rounded down to a multiple of 16, the rest goes to the next prompt
    assert [(s.id, n) for s, n in plan] == [("a", 80), ("b", 8)]
    plan = calc_prefill_per_forward([a, b], 0, 200)
    assert [(s.id, n) for s, n in plan] == [("a", 100), ("b", 30)]


def test_completion_length_predictor():
    means, stds = calc_cumulative_mean_stds([0.1, 0.2, 0.9])
    assert means[0] == pytest.approx(0.4) and means[2] == pytest.approx(0.9) and stds[2] == 0
    t = EarlyStoppingTracker(buffer_size=64, initial_wait=4, std_buffer_scale=0.0, num_buckets=100)
    fresh = _seq(10, max_new=100)
    assert t.predict_completion_length(fresh) == 100          # nothing known yet: assume the limit
    for n in (10, 20, 30, 40):
        done = _seq(10, max_new=100)
        done.output_ids = [0] * n
        t.add_finished_sequences([done])
    assert t.is_warmed_up() and t.buffer_mean() == pytest.approx(0.25)
    assert t.predict_completion_length(fresh) == 25           # mean of all
    late = _seq(10, decode=25, max_new=100)
    assert t.predict_completion_length(late) == 35            # mean of those that ran at least 25
    very_late = _seq(10, decode=60, max_new=100)
    assert t.predict_completion_length(very_late) == 100      # beyond everything seen
    seeded = EarlyStoppingTracker(initial_wait=10, init_mean=0.5, init_std=0.2, std_buffer_scale=0.5)
    assert seeded.predict_completion_length(fresh) == 60


def test_hydragen_grouping():
    ps = 16
    seqs = []
    for i in range(6):
        shared = [1, 2, 3, 4] if i < 4 else [9, 8]
        s = _seq(16 * 6, decode=3, kv=shared + [100 + i, 200 + i, 300 + i], sid=f"q{i}")
        seqs.append(s)
    groups, rest = group_for_hydragen(seqs, ps, min_group_size=3, min_prefix_len=32)
    assert len(groups) == 1 and groups[0].block_ids == [1, 2, 3, 4] and sorted(groups[0].seq_ids) == ["q0", "q1", "q2", "q3"]
    assert sorted(rest) == ["q4", "q5"]
    order = [s.id for s in reorder_decoding_seqs_for_hydragen(list(reversed(seqs)), groups)]
    assert sorted(order[:4]) == ["q0", "q1", "q2", "q3"]
    assert group_for_hydragen(seqs, ps, min_group_size=5, min_prefix_len=32)[0] == []


@pytest.mark.parametrize("steps_ahead,budget", [(1, 4096), (6, 48)])
def test_engine_matches_dense_greedy(steps_ahead, budget):
    model, imodel = build_pair()
    conf = ServerConfig(kv_cache_num_tokens=4096, scheduling_steps_ahead=steps_ahead, max_tokens_per_forward=budget)
    eng = InferenceEngine(imodel, None, model_config(), conf)
    eng.load_state_dict(model.state_dict())
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (5, 33, 70, 17, 40, 9)]
    res = eng.infer_batch([InferenceRequest(i, p, {"max_new_tokens": 20, "top_k": 1}) for i, p in enumerate(prompts)])
    assert [r.id for r in res] == list(range(6))
    for r, p in zip(res, prompts):
        assert r.output_ids[0] == dense_greedy(model, p, 20), r.id
        assert r.finish_reason == ["length"] and len(r.output_logprobs[0]) == 20
    mgr = eng.manager
    mgr.allocator.sanity_checks(set())
    assert mgr.allocator.num_free_blocks() == mgr.num_blocks and mgr.batch_indices.available() == mgr.batch_indices.max_indices
    stats = eng.stats
    assert stats["finished_seqs"] == 6 and stats["decode_tok_per_s"] > 0 and stats["tok_per_forward"] <= budget
    # a second call with shared prefixes reuses cached pages, n > 1 expands into samples
    res2 = eng.infer_batch([InferenceRequest("a", prompts[2] + [1, 2, 3], {"max_new_tokens": 4, "top_k": 1, "n": 2})])
    assert res2[0].num_cached_prompt_tokens == [64, 64] and res2[0].output_ids[0] == res2[0].output_ids[1]
    assert res2[0].output_ids[0] == dense_greedy(model, prompts[2] + [1, 2, 3], 4)


def test_engine_bumps_under_memory_pressure_and_stops_on_tokens():
    model, imodel = build_pair()
    # 12 pages of 16 tokens: four sequences of 20 + 60 tokens cannot all finish at once
    conf = ServerConfig(kv_cache_num_tokens=12 * 16, scheduling_steps_ahead=3, track_early_stopping=False,
                        spec_allocation_target_kv_cache_utilization=4.0)
    eng = InferenceEngine(imodel, None, model_config(), conf)
    eng.load_state_dict(model.state_dict())
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 512, (20,), generator=g).tolist() for _ in range(4)]
    res = eng.infer_batch([InferenceRequest(i, p, {"max_new_tokens": 60, "top_k": 1}) for i, p in enumerate(prompts)])
    assert eng.stats["bumped_seqs"] > 0
    for r, p in zip(res, prompts):
        assert r.output_ids[0] == dense_greedy(model, p, 60), r.id
    eng.manager.allocator.sanity_checks(set())
    want = dense_greedy(model, prompts[0], 10)
    stop = eng.infer_batch([InferenceRequest(0, prompts[0], {"max_new_tokens": 30, "top_k": 1,
                                                              "stop_token_ids": [want[4]]})])[0]
    assert stop.output_ids[0] == want[: want.index(want[4]) + 1] and stop.finish_reason == ["stop_token"]
    # a prompt that can never fit is rejected instead of stalling the loop
    huge = eng.infer_batch([InferenceRequest(0, list(range(250)), {"max_new_tokens": 4})])[0]
    assert huge.finish_reason == ["no_space"] and huge.output_ids == [[]]


def test_engine_with_worker_process_and_lifecycle():
    model, _ = build_pair()
    conf = ServerConfig(kv_cache_num_tokens=2048, scheduling_steps_ahead=4, placement="process")
    eng = InferenceEngine(None, None, model_config(), conf, build_model=build_infer_model_for_worker)
    try:
        eng.load_state_dict(model.state_dict())
        prompt = list(range(3, 40))
        out = eng.infer_batch([InferenceRequest(0, prompt, {"max_new_tokens": 12, "top_k": 1})])[0]
        assert out.output_ids[0] == dense_greedy(model, prompt, 12)
        eng.cleanup()                       # hand the memory back, then take it again with new weights
        eng.initialize()
        eng.load_state_dict(model.state_dict())
        again = eng.infer_batch([InferenceRequest(1, prompt, {"max_new_tokens": 12, "top_k": 1})])[0]
        assert again.output_ids[0] == out.output_ids[0]
    finally:
        eng.shutdown()


def test_cancel_releases_blocks_and_keeps_other_requests_exact():
    """A request cancelled while it runs (and one cancelled before it starts) gives its blocks and
    batch index back, reports finish reason "cancelled" with the tokens received so far, and the
    requests that were not cancelled still match dense greedy decoding."""
    model, imodel = build_pair()
    conf = ServerConfig(kv_cache_num_tokens=4096, scheduling_steps_ahead=2, max_seqs_per_forward=3)
    eng = InferenceEngine(imodel, None, model_config(), conf)
    eng.load_state_dict(model.state_dict())
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (12, 30, 21, 8, 16)]
    calls = {"n": 0}

    def on_step(engine):
        calls["n"] += 1
        if calls["n"] == 3:
            hit = engine.cancel([1, 4])          # 1 is running by now, 4 is still waiting (3 slots)
            assert {s.request_id for s in hit} == {1, 4}

    res = eng.infer_batch([InferenceRequest(i, p, {"max_new_tokens": 24, "top_k": 1}) for i, p in enumerate(prompts)],
                          on_step=on_step)
    by_id = {r.id: r for r in res}
    assert by_id[1].finish_reason == ["cancelled"] and 0 < len(by_id[1].output_ids[0]) < 24
    assert by_id[4].finish_reason == ["cancelled"] and by_id[4].output_ids[0] == []
    assert by_id[1].output_ids[0] == dense_greedy(model, prompts[1], 24)[: len(by_id[1].output_ids[0])]
    for i in (0, 2, 3):
        assert by_id[i].output_ids[0] == dense_greedy(model, prompts[i], 24) and by_id[i].finish_reason == ["length"]
    mgr = eng.manager
    mgr.allocator.sanity_checks(set())
    assert mgr.allocator.num_free_blocks() == mgr.num_blocks
    assert mgr.batch_indices.available() == mgr.batch_indices.max_indices
