"""Actor losses (reference: projects/ppo/variants.py:15-315): clipped PPO with optional
importance-ratio correction against the inference engine's log-probs, the KL-covariance
variant, and the adaptive-entropy variant."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from halite_b200.projects.ppo import math_fn
from halite_b200.projects.ppo.types import ActorLossMixin, CriticMetrics


def response_mask_of(rollouts):
    r = rollouts.batch.response_ids.shape[-1]
    return rollouts.batch.attention_mask[:, -r:].to(torch.float32)


@torch.no_grad()
def compute_critic_metrics(rollouts, response_mask):
    adv_mean = math_fn.masked_mean(rollouts.advantages, response_mask)
    ret_mean = math_fn.masked_mean(rollouts.returns, response_mask)
    return CriticMetrics(
        rewards_mean=rollouts.rewards.sum(-1).mean(),
        advantage_mean=adv_mean,
        advantage_var=math_fn.masked_var(rollouts.advantages, adv_mean, response_mask),
        return_mean=ret_mean,
        return_var=math_fn.masked_var(rollouts.returns, ret_mean, response_mask))


@dataclass
class ClippedSurrogate:
    pg_loss: torch.Tensor
    entropy: torch.Tensor
    ratio: torch.Tensor
    log_ratio: torch.Tensor
    response_mask: torch.Tensor
    pg_clipfrac: torch.Tensor
    approx_kl: torch.Tensor


def ppo_actor_loss(actor, rollouts, clip_low, clip_high, pg_loss_agg, pg_loss_max_tokens,
                   clip_importance_ratio=None):
    log_probs, entropy = actor(rollouts.batch)
    log_ratio = log_probs - rollouts.actor_log_probs
    ratio = log_ratio.exp()
    adv = rollouts.advantages
    unclipped = -adv * ratio
    clipped = -adv * ratio.clamp(1 - clip_low, 1 + clip_high)
    per_token = torch.maximum(unclipped, clipped)
    mask = response_mask_of(rollouts)
    if clip_importance_ratio is not None and rollouts.inference_log_probs is not None:
        # the rollouts were sampled by the inference engine, whose numerics differ slightly
        # from the trainer's: re-weight by trainer / engine probability, truncated
        w = (rollouts.actor_log_probs - rollouts.inference_log_probs).exp().clamp(max=clip_importance_ratio)
        per_token = per_token * w
    loss = math_fn.aggregate_loss(per_token, mask, pg_loss_agg, pg_loss_max_tokens)
    with torch.no_grad():
        clipfrac = math_fn.masked_mean((clipped > unclipped).float(), mask)
        approx_kl = math_fn.masked_mean((ratio - 1) - log_ratio, mask)
    return ClippedSurrogate(loss, entropy, ratio, log_ratio, mask, clipfrac, approx_kl)


@dataclass
class PPOActorLossResults(ActorLossMixin):
    loss: torch.Tensor
    pg_loss: torch.Tensor
    entropy: torch.Tensor
    approx_kl: torch.Tensor
    pg_clipfrac: torch.Tensor
    critic_metrics: CriticMetrics


class PPOActorLoss:
    def __init__(self, clip_low, clip_high, pg_loss_agg, pg_loss_max_tokens=None, clip_importance_ratio=None):
        self.clip_low, self.clip_high = clip_low, clip_high
        self.pg_loss_agg = pg_loss_agg
        self.pg_loss_max_tokens = pg_loss_max_tokens
        self.clip_importance_ratio = clip_importance_ratio

    def compute_actor_loss(self, actor, rollouts):
        s = ppo_actor_loss(actor, rollouts, self.clip_low, self.clip_high, self.pg_loss_agg,
                           self.pg_loss_max_tokens, self.clip_importance_ratio)
        entropy = s.entropy
        if entropy is not None and entropy.dim() > 0:
            entropy = math_fn.masked_mean(entropy.detach(), s.response_mask)
        return PPOActorLossResults(loss=s.pg_loss, pg_loss=s.pg_loss.detach(), entropy=entropy,
                                   approx_kl=s.approx_kl, pg_clipfrac=s.pg_clipfrac,
                                   critic_metrics=compute_critic_metrics(rollouts, s.response_mask))


@dataclass
class PPOKLCovActorLossResults(ActorLossMixin):
    loss: torch.Tensor
    pg_loss: torch.Tensor
    entropy: torch.Tensor
    approx_kl: torch.Tensor
    critic_metrics: CriticMetrics


class PPOKLCovActorLoss:
    """Unclipped policy gradient; the fraction `select_ratio` of response tokens with the largest
    advantage / log-prob covariance additionally pays `kl_coef * |log ratio|`."""

    def __init__(self, pg_loss_agg, pg_loss_max_tokens, kl_coef, select_ratio):
        self.pg_loss_agg = pg_loss_agg
        self.pg_loss_max_tokens = pg_loss_max_tokens
        self.kl_coef = kl_coef
        self.select_ratio = select_ratio

    def compute_actor_loss(self, actor, rollouts):
        log_probs, entropy = actor(rollouts.batch)
        log_ratio = log_probs - rollouts.actor_log_probs
        ratio = log_ratio.exp()
        mask = response_mask_of(rollouts)
        per_token = -rollouts.advantages * ratio
        valid = mask > 0
        n_valid = int(valid.sum())
        if self.select_ratio > 0 and n_valid > 0:
            adv = rollouts.advantages[valid].detach()
            lp = log_probs[valid].detach()
            cov = (adv - adv.mean()) * (lp - lp.mean())
            k = max(1, int(n_valid * min(self.select_ratio, 1.0)))
            top = torch.topk(cov, k).indices
            flat = torch.nonzero(valid.reshape(-1), as_tuple=True)[0][top]
            pick = torch.zeros_like(valid.reshape(-1))
            pick[flat] = True
            pick = pick.view_as(valid)
            per_token = torch.where(pick, per_token + self.kl_coef * log_ratio.abs(), per_token)
        loss = math_fn.aggregate_loss(per_token, mask, self.pg_loss_agg, self.pg_loss_max_tokens)
        with torch.no_grad():
            approx_kl = math_fn.masked_mean((ratio - 1) - log_ratio, mask)
            ent = math_fn.masked_mean(entropy, mask) if entropy is not None else None
        return PPOKLCovActorLossResults(loss=loss, pg_loss=loss.detach(), entropy=ent, approx_kl=approx_kl,
                                        critic_metrics=compute_critic_metrics(rollouts, mask))


@dataclass
class PPOAdaptiveEntropyActorLossResults(ActorLossMixin):
    loss: torch.Tensor
    pg_loss: torch.Tensor
    entropy: torch.Tensor
    approx_kl: torch.Tensor
    pg_clipfrac: torch.Tensor
    entropy_coef: float
    critic_metrics: CriticMetrics


class PPOAdaptiveEntropyActorLoss:
    """Clipped PPO minus `entropy_coef * entropy`; the coefficient steps up while the measured
    entropy is below `target_entropy` and down otherwise, within [min, max]."""

    def __init__(self, clip_low, clip_high, pg_loss_agg, pg_loss_max_tokens, init_entropy_coef,
                 min_entropy_coef, max_entropy_coef, entropy_coef_update_size, target_entropy,
                 clip_importance_ratio=None):
        self.clip_low, self.clip_high = clip_low, clip_high
        self.pg_loss_agg = pg_loss_agg
        self.pg_loss_max_tokens = pg_loss_max_tokens
        self.clip_importance_ratio = clip_importance_ratio
        self.entropy_coef = init_entropy_coef
        self.min_entropy_coef = min_entropy_coef
        self.max_entropy_coef = max_entropy_coef
        self.entropy_coef_update_size = entropy_coef_update_size
        self.target_entropy = target_entropy

    def update_entropy_coef(self, entropy: float):
        step = self.entropy_coef_update_size if entropy < self.target_entropy else -self.entropy_coef_update_size
        self.entropy_coef = min(max(self.entropy_coef + step, self.min_entropy_coef), self.max_entropy_coef)

    def compute_actor_loss(self, actor, rollouts):
        s = ppo_actor_loss(actor, rollouts, self.clip_low, self.clip_high, self.pg_loss_agg,
                           self.pg_loss_max_tokens, self.clip_importance_ratio)
        entropy = math_fn.masked_mean(s.entropy, s.response_mask)
        self.update_entropy_coef(float(entropy.detach()))
        loss = s.pg_loss - self.entropy_coef * entropy
        return PPOAdaptiveEntropyActorLossResults(
            loss=loss, pg_loss=s.pg_loss.detach(), entropy=entropy.detach(), approx_kl=s.approx_kl,
            pg_clipfrac=s.pg_clipfrac, entropy_coef=self.entropy_coef,
            critic_metrics=compute_critic_metrics(rollouts, s.response_mask))
