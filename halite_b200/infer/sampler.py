"""Next-token sampling (reference: infer/engine/sampler.py:12-60): NaN guard, greedy argmax or
temperature -> (top-k / top-p / min-p filter) -> categorical draw; returns the chosen ids and
their log-probability under the temperature-scaled distribution.

Unfiltered sampling (the RL rollout case: top_p = 1, top_k off) draws by the Gumbel-max trick,
which needs one pass over the vocabulary and no sort; the sm_100a `sample_gumbel` kernel does
softmax statistics, noise, argmax and the log-prob in that single pass.
"""

from __future__ import annotations

import torch

from halite_b200 import ops


class Sampler:
    def __init__(self, use_nan_detection=True, seed=0):
        self.use_nan_detection = use_nan_detection
        self.seed = seed
        self._calls = 0

    def forward(self, logits, sampling, generator=None):
        """logits [B, V] fp32 -> (ids int64 [B], logprobs fp32 [B])."""
        logits = logits.float()
        if self.use_nan_detection and not logits.is_cuda:
            nan = torch.isnan(logits)
            if nan.any():
                logits = torch.where(nan, torch.full_like(logits, -1e5), logits)
        if sampling.is_all_greedy:
            ids = logits.argmax(-1)
            lp = torch.log_softmax(logits, -1).gather(-1, ids.unsqueeze(-1)).squeeze(-1)
            return ids, lp
        if not (sampling.need_top_k_top_p or sampling.need_min_p_sampling):
            return self._gumbel(logits, sampling, generator)
        return self._filtered(logits, sampling, generator)

    __call__ = forward

    def _gumbel(self, logits, sampling, generator):
        greedy = (sampling.top_ks <= 1)
        if logits.is_cuda and not ops.force_reference() and generator is None:
            self._calls += 1
            ids, lp = ops.ext().sample_gumbel(logits.contiguous(), sampling.temperatures.view(-1).contiguous(),
                                              greedy.contiguous(), self.seed, self._calls)
            return ids, lp
        scaled = logits / sampling.temperatures
        logp = torch.log_softmax(scaled, -1)
        u = torch.rand(scaled.shape, device=scaled.device, generator=generator).clamp_(1e-10, 1.0)
        noisy = scaled - torch.log(-torch.log(u))
        noisy = torch.where(greedy.unsqueeze(-1), scaled, noisy)
        ids = noisy.argmax(-1)
        return ids, logp.gather(-1, ids.unsqueeze(-1)).squeeze(-1)

    def _filtered(self, logits, sampling, generator):
        scaled = logits / sampling.temperatures
        probs = torch.softmax(scaled, -1)
        sorted_p, order = probs.sort(-1, descending=True)
        cum = sorted_p.cumsum(-1)
        ranks = torch.arange(probs.shape[-1], device=probs.device).unsqueeze(0)
        keep = ranks < sampling.top_ks.unsqueeze(-1)
        # top-p: keep the smallest set whose mass reaches top_p (the token crossing it stays)
        keep &= (cum - sorted_p) < sampling.top_ps.unsqueeze(-1)
        if sampling.need_min_p_sampling:
            keep &= sorted_p >= sampling.min_ps.unsqueeze(-1) * sorted_p[:, :1]
        keep[:, 0] = True
        filt = torch.where(keep, sorted_p, torch.zeros_like(sorted_p))
        filt = filt / filt.sum(-1, keepdim=True)
        pick = torch.multinomial(filt, 1, generator=generator)
        ids = order.gather(-1, pick).squeeze(-1)
        lp = torch.log(probs.gather(-1, ids.unsqueeze(-1)).squeeze(-1))
        return ids, lp
