"""PPO / GRPO trainer pieces (reference: projects/ppo/trainer.py:12-355): batch building from
rollouts, KL penalty, GAE and group-relative advantages, the trainer that scores rollouts and
computes actor (and critic) losses."""

from __future__ import annotations

import torch
from torch.nn import functional as F

from halite_b200 import ops
from halite_b200.projects.ppo import math_fn
from halite_b200.projects.ppo.types import Batch, RolloutBatch


def build_batch_from_rollouts(rollouts, offset=0, pad_id=-1, device=None):
    """Prompts left-padded to a common boundary, responses right-padded after it; position ids
    count real tokens; rewards are right-padded token rewards; ids group samples of one prompt."""
    group = {}
    ids = [group.setdefault(r.id, len(group)) for r in rollouts]
    n = len(rollouts)
    p_len = [len(r.input_ids) for r in rollouts]
    r_len = [len(r.output_ids) for r in rollouts]
    P, R = max(p_len), max(r_len)
    input_ids = torch.zeros(n, P + R, dtype=torch.int64)
    attention_mask = torch.zeros_like(input_ids)
    position_ids = torch.zeros_like(input_ids)
    response_ids = torch.full((n, R), pad_id, dtype=torch.int64)
    has_lp = rollouts[0].output_logprobs is not None
    response_logprobs = torch.zeros(n, R, dtype=torch.float32) if has_lp else None
    reward_rows = [torch.as_tensor(r.rewards).reshape(-1) for r in rollouts]
    rewards = reward_rows[0].new_zeros(n, max(x.shape[-1] for x in reward_rows))
    for i, r in enumerate(rollouts):
        lo, mid, hi = P - p_len[i], P, P + r_len[i]
        input_ids[i, lo:mid] = torch.as_tensor(r.input_ids)
        resp = torch.as_tensor(r.output_ids, dtype=torch.int64)
        input_ids[i, mid:hi] = resp
        attention_mask[i, lo:hi] = 1
        position_ids[i, lo:hi] = torch.arange(hi - lo)
        response_ids[i, : r_len[i]] = resp
        rewards[i, : reward_rows[i].shape[-1]] = reward_rows[i]
        if has_lp:
            response_logprobs[i, : r_len[i]] = torch.as_tensor(r.output_logprobs, dtype=torch.float32)
    temps = [r.sampling_params.get("temperature", 1.0) for r in rollouts]
    temperatures = temps[0] if all(t == temps[0] for t in temps) else torch.tensor(temps)
    to = lambda t: t.to(device) if (device is not None and isinstance(t, torch.Tensor)) else t
    return Batch(to(input_ids), to(response_ids), to(attention_mask), to(position_ids), to(rewards),
                 to(torch.tensor(ids)), to(torch.tensor(p_len)), to(torch.tensor(r_len)),
                 to(temperatures), to(response_logprobs))


def log_probs_from_logits(logits, labels, ignore_index, temperature=1.0):
    if isinstance(temperature, torch.Tensor):
        logits = logits / temperature.reshape(-1, 1, 1)
    elif temperature != 1.0:
        logits = logits / temperature
    return -F.cross_entropy(logits.permute(0, 2, 1), labels, reduction="none", ignore_index=ignore_index)


def entropy_from_logits(logits, temperature=1.0):
    if isinstance(temperature, torch.Tensor):
        logits = logits / temperature.reshape(-1, 1, 1)
    elif temperature != 1.0:
        logits = logits / temperature
    lp = torch.log_softmax(logits, -1)
    return -(lp.exp() * lp).sum(-1)


def compute_approx_kl(log_probs, ref_log_probs):
    """The non-negative, low-variance estimator exp(d) - 1 - d of KL(ref || actor) per token."""
    d = log_probs - ref_log_probs
    return d.exp() - 1 - d


class KLPenalty:
    def __init__(self, kl_coef, method="approx"):
        self.kl_coef = kl_coef
        self.method = method

    def __call__(self, rewards, actor_out, ref_out):
        kl = compute_approx_kl(actor_out, ref_out) if self.method == "approx" else actor_out - ref_out
        return rewards - self.kl_coef * kl


@torch.no_grad()
def compute_ppo_advantage(rewards, mask, values, gamma, lam, reward_whitening=True,
                          advantage_whitening=True, **unused):
    """Generalised advantage estimation over the response window. One reverse-scan kernel on
    the GPU; padding positions (mask == 0) are skipped by the scan."""
    mask_f = mask.to(torch.float32) if mask is not None else None
    if reward_whitening:
        rewards = math_fn.whitening(rewards, shift_mean=False, mask=mask_f)
    advantages, returns = ops.gae(rewards.float(), values.float(), gamma, lam, mask_f)
    if advantage_whitening:
        advantages = math_fn.whitening(advantages, shift_mean=True, mask=mask_f)
        if mask_f is not None:
            advantages = advantages * mask_f
    return advantages, returns


@torch.no_grad()
def compute_grpo_advantage(rewards, mask, group_ids, std_normalize=True, eps=1e-6, **unused):
    """Sequence reward minus the mean over samples of the same prompt (optionally divided by the
    group's standard deviation), broadcast over the response tokens."""
    total = rewards.sum(-1)
    _, idx = group_ids.unique(sorted=True, return_inverse=True)
    count = torch.bincount(idx).to(total.dtype)
    mean = torch.bincount(idx, weights=total) / count
    mean = torch.where(count == 1, torch.zeros_like(mean), mean)
    adv = total - mean[idx]
    if std_normalize:
        var = torch.bincount(idx, weights=adv.square()) / (count - 1).clamp(min=1)
        std = torch.where(count == 1, torch.ones_like(var), var.sqrt())
        adv = adv / (std[idx] + eps)
    adv = adv.unsqueeze(-1) * mask
    return adv, adv


class PPOTrainer:
    def __init__(self, actor, advantage_fn, actor_loss, ref=None, penalty_fn=None, critic=None,
                 log_probs_batch_size=None, device=None, value_clip=0.2):
        self.actor = actor
        self.advantage_fn = advantage_fn
        self.actor_loss = actor_loss
        self.ref = ref
        self.penalty_fn = penalty_fn
        self.critic = critic
        self.log_probs_batch_size = log_probs_batch_size
        self.device = device
        self.pad_id = -1
        self.value_clip = value_clip

    def compute_log_probs(self, batch):
        actor_out, actor_entropy = self.actor(batch)
        ref_out = self.ref(batch)[0] if self.ref is not None else None
        critic_out = self.critic(batch) if self.critic is not None else None
        return actor_out, actor_entropy, ref_out, critic_out

    @torch.no_grad()
    def compute_advantage(self, rollouts):
        batch = build_batch_from_rollouts(rollouts, offset=-1, pad_id=self.pad_id, device=self.device)
        parts = batch.split(self.log_probs_batch_size) if self.log_probs_batch_size else [batch]
        cols = [[], [], [], []]
        for micro in parts:
            for col, val in zip(cols, self.compute_log_probs(micro)):
                if val is not None:
                    col.append(val)
        actor_out, actor_entropy, ref_out, critic_out = (torch.cat(c, 0) if c else None for c in cols)
        rewards = batch.rewards
        if self.penalty_fn is not None:
            rewards = self.penalty_fn(rewards, actor_out, ref_out)
        r = batch.response_ids.shape[-1]
        mask = batch.attention_mask[:, -r:]
        advantages, returns = self.advantage_fn(rewards, mask, values=critic_out, group_ids=batch.ids)
        return RolloutBatch(rollouts=rollouts, rewards=rewards, batch=batch, advantages=advantages,
                            returns=returns, actor_log_probs=actor_out, actor_entropy=actor_entropy,
                            inference_log_probs=batch.response_logprobs, values=critic_out)

    def compute_actor_loss(self, rollouts):
        return self.actor_loss.compute_actor_loss(self.actor, rollouts)

    def compute_critic_loss(self, rollouts):
        """Clipped value loss: 0.5 * mean(max((v - R)^2, (clip(v, v_old +- c) - R)^2))."""
        values = self.critic(rollouts.batch)
        r = rollouts.batch.response_ids.shape[-1]
        mask = rollouts.batch.attention_mask[:, -r:].to(torch.float32)
        returns = rollouts.returns
        loss = (values - returns).square()
        clipfrac = torch.zeros((), device=values.device)
        if rollouts.values is not None and self.value_clip is not None:
            old = rollouts.values
            clipped = old + (values - old).clamp(-self.value_clip, self.value_clip)
            loss2 = (clipped - returns).square()
            clipfrac = math_fn.masked_mean((loss2 > loss).float(), mask).detach()
            loss = torch.maximum(loss, loss2)
        loss = 0.5 * math_fn.masked_mean(loss, mask)
        return loss, {"critic/loss": loss.detach(), "critic/clipfrac": clipfrac,
                      "critic/value_mean": math_fn.masked_mean(values.detach(), mask)}
