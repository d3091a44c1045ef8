"""PPO / GRPO pipeline with deterministic mocks (pattern of the reference's test/test_ppo.py):
rollout expansion, token rewards, batch padding, group-relative advantages and the exact
gradient of the token-sum clipped loss; plus GAE, whitening, the critic loss and the
real actor wrapper on a tiny model."""

import uuid
from functools import partial

import pytest
import torch
from torch.nn import functional as F

from halite_b200.infer.types import InferenceResult
from halite_b200.projects.common.rollout import Handler, RewardRegistry, Rollout, RolloutGenerator
from halite_b200.projects.common.rollout_fn import Compose, ToTokenReward, WeightedSum
from halite_b200.projects.ppo import math_fn
from halite_b200.projects.ppo.trainer import (KLPenalty, PPOTrainer, build_batch_from_rollouts,
                                              compute_grpo_advantage, compute_ppo_advantage,
                                              entropy_from_logits, log_probs_from_logits)
from halite_b200.projects.ppo.variants import PPOActorLoss, PPOAdaptiveEntropyActorLoss, PPOKLCovActorLoss


class EngineMock:
    def initialize(self):
        pass

    def infer_batch(self, requests):
        return [
            InferenceResult(id=requests[0].id, input_ids=[1, 2, 3, 4, 5],
                            output_ids=[[6, 7, 8], [6, 7, 8, 9, 10], [1, 2]]),
            InferenceResult(id=requests[1].id, input_ids=[6, 7, 8],
                            output_ids=[[1, 2, 3, 4, 5], [6, 7], [8, 9, 10]]),
        ]


class ActorMock:
    """Logits arange / 100 over [B, L, 11]; keeps them so the test can read the gradient."""

    def __call__(self, data):
        r = data.response_ids.shape[-1]
        logits = (torch.arange(data.input_ids.numel() * 11, dtype=torch.float32)
                  .reshape(*data.input_ids.shape, 11) / 100).requires_grad_(True)
        self.logits = logits
        window = logits[:, r - 1:-1]
        return (log_probs_from_logits(window, data.response_ids, -1, data.temperatures),
                entropy_from_logits(window, data.temperatures))


def make_rollouts():
    gen = RolloutGenerator(EngineMock(), RewardRegistry(
        Handler("mock", lambda outs: torch.arange(1, len(outs) + 1, dtype=torch.float32), args=("output_ids",)),
        postprocess=Compose(ToTokenReward("output_ids", "mock", "token_rewards"))))
    gen.initialize()
    return gen.generate([
        Rollout(id=uuid.uuid4().hex, input_ids=[1, 2, 3, 4, 5], type="math",
                sampling_params={"max_new_tokens": 512, "n": 4}, state={"input_text": "a"}),
        Rollout(id=uuid.uuid4().hex, input_ids=[6, 7, 8], type="arithmetic",
                sampling_params={"max_new_tokens": 512, "n": 4}, state={"input_text": "b"}),
    ])


def test_grpo_pipeline_matches_hand_computation():
    rollouts = make_rollouts()
    actor = ActorMock()
    trainer = PPOTrainer(actor, compute_grpo_advantage,
                         PPOActorLoss(clip_low=0.2, clip_high=0.2, pg_loss_agg="token-sum", pg_loss_max_tokens=4096))
    rb = trainer.compute_advantage(rollouts)
    res = trainer.compute_actor_loss(rb)
    want_rewards = torch.tensor([[0, 0, 1, 0, 0], [0, 0, 0, 0, 2], [0, 3, 0, 0, 0],
                                 [0, 0, 0, 0, 4], [0, 5, 0, 0, 0], [0, 0, 6, 0, 0]], dtype=torch.float32)
    assert torch.allclose(rb.rewards, want_rewards)
    want_ids = torch.tensor([[1, 2, 3, 4, 5, 6, 7, 8, 0, 0], [1, 2, 3, 4, 5, 6, 7, 8, 9, 10],
                             [1, 2, 3, 4, 5, 1, 2, 0, 0, 0], [0, 0, 6, 7, 8, 1, 2, 3, 4, 5],
                             [0, 0, 6, 7, 8, 6, 7, 0, 0, 0], [0, 0, 6, 7, 8, 8, 9, 10, 0, 0]])
    assert torch.equal(rb.batch.input_ids, want_ids)
    assert rb.batch.position_ids[3].tolist() == [0, 0, 0, 1, 2, 3, 4, 5, 6, 7]
    want_adv = torch.tensor([[-1, -1, -1, 0, 0], [0, 0, 0, 0, 0], [1, 1, 0, 0, 0],
                             [-1, -1, -1, -1, -1], [0, 0, 0, 0, 0], [1, 1, 1, 0, 0]], dtype=torch.float32)
    assert torch.allclose(rb.advantages, want_adv, atol=1e-5)
    res.loss.backward()
    # independent restatement of the token-sum loss at ratio == 1
    logits = (torch.arange(rb.batch.input_ids.numel() * 11, dtype=torch.float32)
              .reshape(*rb.batch.input_ids.shape, 11) / 100).requires_grad_(True)
    r = rb.batch.response_ids.shape[-1]
    lp = log_probs_from_logits(logits[:, r - 1:-1], rb.batch.response_ids, -1, rb.batch.temperatures)
    mask = rb.batch.attention_mask[:, -r:]
    ref = torch.sum(-rb.advantages * (lp - lp.detach()) * mask) / (4096 * lp.shape[0])
    ref.backward()
    assert torch.allclose(actor.logits.grad, logits.grad, atol=1e-9)
    metrics = res.metric_dict()
    assert {"actor/loss", "actor/pg_loss", "actor/approx_kl", "critic/rewards_mean"} <= set(metrics)
    assert abs(float(metrics["actor/approx_kl"])) < 1e-6


def test_batch_split_and_other_losses():
    rollouts = make_rollouts()
    trainer = PPOTrainer(ActorMock(), partial(compute_grpo_advantage, std_normalize=False),
                         PPOAdaptiveEntropyActorLoss(0.2, 0.2, "token-mean", None, 0.0, 0.0, 0.01, 0.001, 5.0),
                         log_probs_batch_size=2)
    rb = trainer.compute_advantage(rollouts)
    parts = rb.split(2)
    assert len(parts) == 3 and parts[1].batch.input_ids.shape == (2, 10) and len(parts[2].rollouts) == 2
    res = trainer.compute_actor_loss(parts[0])
    assert res.entropy_coef == pytest.approx(0.001)           # entropy below target: coefficient steps up
    res.loss.backward()
    klcov = PPOKLCovActorLoss("token-mean", None, kl_coef=1.0, select_ratio=0.5)
    out = klcov.compute_actor_loss(ActorMock(), parts[1])
    assert torch.isfinite(out.loss)


def test_gae_matches_loop_and_whitening_mask():
    torch.manual_seed(0)
    rewards, values = torch.randn(5, 9), torch.randn(5, 9)
    adv, ret = compute_ppo_advantage(rewards, None, values, 0.99, 0.95, reward_whitening=False,
                                     advantage_whitening=False)
    last, rows = 0, []
    for t in reversed(range(9)):
        nxt = values[:, t + 1] if t < 8 else 0.0
        delta = rewards[:, t] + 0.99 * nxt - values[:, t]
        last = delta + 0.99 * 0.95 * last
        rows.append(last)
    want = torch.stack(rows[::-1], 1)
    assert torch.allclose(adv, want, atol=1e-5) and torch.allclose(ret, want + values, atol=1e-5)
    mask = torch.ones(5, 9)
    mask[:, 6:] = 0
    adv_m, _ = compute_ppo_advantage(rewards, mask, values, 1.0, 0.95)
    assert (adv_m[:, 6:] == 0).all()
    inside = adv_m[:, :6]
    assert abs(inside.mean()) < 1e-5 and abs(inside.std(correction=0) - 1) < 1e-3
    w = math_fn.whitening(rewards, shift_mean=False, mask=mask)
    assert torch.isfinite(w).all()
    pen = math_fn.truncate_penalty(torch.tensor([[1, 2, 9], [1, 2, 3]]), torch.tensor([1.0, 1.0]), 9, -5.0)
    assert pen.tolist() == [1.0, -5.0]


def test_kl_penalty_and_weighted_rewards():
    a, b = torch.tensor([[0.0, -1.0]]), torch.tensor([[0.0, -0.5]])
    out = KLPenalty(0.05)(torch.ones(1, 2), a, b)
    d = a - b
    assert torch.allclose(out, 1 - 0.05 * (d.exp() - 1 - d))
    assert torch.allclose(KLPenalty(0.05, "plain")(torch.ones(1, 2), a, b), 1 - 0.05 * d)
    reg = RewardRegistry(
        Handler("len", lambda o: torch.tensor([float(len(x)) for x in o]), args=("output_ids",)),
        Handler("only_math", lambda o: torch.ones(len(o)), args=("output_ids",), targets=("math",), reward_padding=-1),
        postprocess=Compose(WeightedSum("total", len=1.0, only_math=10.0)))
    rs = [Rollout("a", [1], [1, 2, 3], type="math"), Rollout("b", [1], [4], type="code")]
    reg(rs)
    assert float(rs[0].rewards) == 13.0 and float(rs[1].rewards) == -9.0
    assert float(rs[1].rewards_dict["only_math"]) == -1.0


def test_real_actor_wrapper_and_critic(zoo):
    """UnpaddedModel on a tiny decoder: log-probs / entropy equal a padded dense evaluation;
    critic loss with value clipping runs and has gradients."""
    from halite_b200.conf import instantiate
    from halite_b200.projects.ppo.model import ScalarHead, UnpaddedModel, ValueModel
    from tests.conftest import tiny_llama_conf

    torch.manual_seed(0)
    model = instantiate(tiny_llama_conf(zoo, n_layers=2))
    model.init_weights()
    g = torch.Generator().manual_seed(0)
    rollouts = []
    for i, (p, r) in enumerate([(5, 7), (9, 3), (4, 9)]):
        ro = Rollout(id=str(i), input_ids=torch.randint(0, 1024, (p,), generator=g).tolist(),
                     output_ids=torch.randint(0, 1024, (r,), generator=g).tolist(),
                     sampling_params={"temperature": 0.7})
        ro.rewards = torch.zeros(r)
        ro.rewards[-1] = float(i)
        rollouts.append(ro)
    batch = build_batch_from_rollouts(rollouts)
    logp, ent = UnpaddedModel(model)(batch)
    R = batch.response_ids.shape[-1]
    for i, ro in enumerate(rollouts):
        seq = torch.tensor([ro.input_ids + ro.output_ids])
        logits = model(seq).logits[0].float() / 0.7
        lp = torch.log_softmax(logits, -1)
        n_in, n_out = len(ro.input_ids), len(ro.output_ids)
        want = lp[n_in - 1:-1].gather(-1, torch.tensor(ro.output_ids)[:, None]).squeeze(-1)
        assert torch.allclose(logp[i, :n_out], want, atol=1e-4)
        want_ent = -(lp.exp() * lp).sum(-1)[n_in - 1:-1]
        assert torch.allclose(ent[i, :n_out], want_ent, atol=1e-4)
    critic_body = instantiate(tiny_llama_conf(zoo, n_layers=1, use_head=False))
    critic_body.init_weights()
    head = ScalarHead(256)
    head.init_weights()
    critic = ValueModel(critic_body, head)
    trainer = PPOTrainer(UnpaddedModel(model), partial(compute_ppo_advantage, gamma=1.0, lam=0.95),
                         PPOActorLoss(0.2, 0.2, "token-mean"), critic=critic)
    rb = trainer.compute_advantage(rollouts)
    assert rb.values.shape == (3, R) and rb.advantages.shape == (3, R)
    loss, metrics = trainer.compute_critic_loss(rb)
    loss.backward()
    assert head.linear.weight.grad is not None and torch.isfinite(loss)
    assert critic.score(batch).shape == (3,)


def test_async_rollout_primitives():
    import threading

    from halite_b200.projects.common.rollout_async import ReplayBuffer, TensorSpec, chunk_list, get_peer_ranks

    assert chunk_list(list(range(7)), 3) == [[0, 1, 2], [3, 4], [5, 6]]
    assert get_peer_ranks(1, 2, 4) == [2, 3] and get_peer_ranks(3, 4, 2) == [] and get_peer_ranks(1, 4, 4) == [1]
    assert get_peer_ranks(3, 4, 2, overlap_targets=True) == [1]
    spec = TensorSpec.from_tensor("w", torch.zeros(2, 3, dtype=torch.bfloat16))
    assert spec.empty("cpu").shape == (2, 3) and spec.dtype == torch.bfloat16
    buf = ReplayBuffer(capacity=3, max_staleness=1)
    for v in range(5):
        buf.put(v, [f"r{v}"])
    assert len(buf) == 3 and buf.dropped == 2                       # capacity
    assert buf.get(current_version=4)[0] == 3 and buf.dropped == 3  # version 2 was too stale
    assert buf.get(current_version=4)[0] == 4
    with pytest.raises(TimeoutError):
        buf.get(4, timeout=0.05)
    threading.Timer(0.05, lambda: buf.put(9, ["late"])).start()
    assert buf.get(9, timeout=5) == (9, ["late"])


def test_ppo_iteration_benchmark_runs_four_models():
    """Actor, critic, reference and reward model through one timed iteration (tiny widths)."""
    import os

    from benchmarks import bench_ppo_iter as bench_iter

    conf = os.path.join(os.path.dirname(os.path.abspath(__file__)), "configs/tiny_ppo_models.py")
    out = bench_iter.main(["--conf", conf, "--prompts", "8", "--prompt-len", "12", "--new-tokens", "10",
                           "--microbatch", "2", "--iters", "1", "--warmup", "0", "--device", "cpu"])
    assert out["sampled_tokens_per_iteration_per_rank"] == 80 and out["value"] > 0
    assert set(out["phases_s_per_iteration"]) == {"weight_sync", "rollout_and_reward_model", "reward_model",
                                                  "engine_release", "logprobs_values_gae", "update"}
