"""Rollout preprocessors and reward post-processors (reference: projects/common/rollout_fn.py)."""

from __future__ import annotations

import torch


class Detokenize:
    def __init__(self, tokenizer, keys=("output_ids",), output_keys=("output_texts",), **tokenizer_kwargs):
        self.tokenizer = tokenizer
        self.keys = keys
        self.output_keys = output_keys
        self.tokenizer_kwargs = tokenizer_kwargs

    def __call__(self, rollout):
        for i, key in enumerate(self.keys):
            if not rollout.has_field(key):
                continue
            target = self.output_keys[i] if self.output_keys else key
            rollout.set_field(target, self.tokenizer.decode(rollout.get_field(key), **self.tokenizer_kwargs))
        return rollout


class Compose:
    def __init__(self, *postprocessors):
        self.postprocessors = postprocessors

    def __call__(self, rewards_dict, rollouts):
        rewards = None
        for fn in self.postprocessors:
            rewards, rewards_dict = fn(rewards_dict, rollouts)
        return rewards, rewards_dict


class WeightedSum:
    def __init__(self, output_key, /, **weights):
        self.output_key = output_key
        self.weights = weights

    def __call__(self, rewards_dict, rollouts):
        total = sum(rewards_dict[k] * w for k, w in self.weights.items())
        return total, {**rewards_dict, self.output_key: total}


class ToTokenReward:
    """Scalar reward per rollout -> [n, T] with the scalar on the last token of the sample."""

    def __init__(self, sample_key, reward_key, output_key):
        self.sample_key = sample_key
        self.reward_key = reward_key
        self.output_key = output_key

    def __call__(self, rewards_dict, rollouts):
        lengths = [len(r.get_field(self.sample_key)) for r in rollouts]
        scalar = rewards_dict[self.reward_key]
        out = scalar.new_zeros(len(rollouts), max(lengths))
        rows = torch.arange(len(rollouts))
        out[rows, torch.tensor(lengths) - 1] = scalar
        return out, {**rewards_dict, self.output_key: out}
