"""Reward functions of the reasoning experiments, built the way an experiment builds them
(recorded in a config file, instantiated at run time), and the fork-based timeout."""

import os
import time

import pytest
import torch

from halite_b200.conf import external, instantiate
from halite_b200.conf.loader import load_module
from halite_b200.projects.rewards.math_verify import TimeoutException, _fallback_equal, math_metric, timeout
from tests.helpers import ROOT

rewards = load_module(os.path.join(ROOT, "configs/reasoning/rewards.py"))


def test_math_verify_and_format_rewards():
    mv = instantiate(external[rewards.MathVerify]())
    got = mv(["<think>x</think> <answer>\\frac{1}{2}</answer>", "<answer>3</answer>", "no answer tag"],
             ["$\\frac{1}{2}$", "$4$", "$1$"])
    assert got.tolist() == [1.0, 0.0, 0.0]
    fr = instantiate(external[rewards.FormatReward]())
    assert fr(["a</think> <answer>1</answer>", "<answer>1</answer>"]).tolist() == [1.0, 0.0]
    forked = instantiate(external[rewards.MathVerify](multiprocess_mode=True, timeout_seconds=30))
    assert forked(["<answer>0.5</answer>"], ["$\\frac{1}{2}$"]).tolist() == [1.0]


def test_metric_fallback_and_timeout():
    assert _fallback_equal("\\frac{1}{2}", "\\boxed{0.5}", 6) and not _fallback_equal("2", "3", 6)
    score, strings = math_metric()(["7"], ["the answer is 7"])
    assert score == 1.0 and strings is not None

    @timeout(0.3)
    def slow():
        time.sleep(5)

    @timeout(5)
    def fine(x):
        return x + 1

    @timeout(5)
    def broken():
        raise KeyError("boom")

    with pytest.raises(TimeoutException):
        slow()
    assert fine(2) == 3
    with pytest.raises(KeyError):
        broken()


def test_reasoning_experiment_config_loads():
    """configs/reasoning/math.py validates against the PPO schema once an actor folder exists."""
    mod = load_module(os.path.join(ROOT, "configs/reasoning/math.py"))
    assert mod.conf.training.ppo_microbatch_size == 4 and "problem" in mod.template
    assert mod.conf.data.train.shards["EleutherAI_hendrycks_math"]["algebra-train-1-of-1.bag"] == 1744
