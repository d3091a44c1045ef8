"""Model wrappers used by the PPO trainer (reference: projects/ppo/model.py:18-96).

`UnpaddedModel` returns per-token log-probabilities of the taken tokens and entropies over
the response window. Padding is removed before the transformer runs (packed tokens +
cumulative lengths), and the head is applied through `ops.logprob_entropy`, so neither the
padded activations nor the [tokens, vocab] logits are materialised. `ValueModel` wraps a
decoder without LM head plus a scalar head (critic and reward models).
"""

from __future__ import annotations

import torch
from torch import nn

from halite_b200 import ops
from halite_b200.models.attention import build_unpad_params, pad_input, unpad_input


class ModelWrapper:
    def __init__(self, model):
        self.model = model

    def parameters(self):
        return self.model.parameters()

    def named_parameters(self):
        return self.model.named_parameters()

    def state_dict(self, *args, **kwargs):
        return self.model.state_dict(*args, **kwargs)

    def load_state_dict(self, *args, **kwargs):
        return self.model.load_state_dict(*args, **kwargs)

    def train(self, mode=True):
        self.model.train(mode)
        return self

    def eval(self):
        return self.train(False)


def _head_weight(model):
    head = getattr(model, "head", None)
    if head is None:
        raise ValueError("the actor model needs a vocabulary head")
    return head.weight


class UnpaddedModel(ModelWrapper):
    def __init__(self, model, pad_id: int = -1, calc_log_probs: bool = True, calc_entropy: bool = True):
        super().__init__(model)
        self.pad_id = pad_id
        self.calc_log_probs = calc_log_probs
        self.calc_entropy = calc_entropy

    def hidden_states(self, batch):
        """Final hidden states of the packed (padding-free) tokens: [total, dim], params."""
        params = build_unpad_params(batch.attention_mask)
        ids = unpad_input(batch.input_ids.unsqueeze(-1), params).squeeze(-1)
        pos = unpad_input(batch.position_ids.unsqueeze(-1), params).squeeze(-1)
        head, self.model.head = self.model.head, None
        try:
            out = self.model(ids, position_ids=pos, unpad_params=params)
        finally:
            self.model.head = head
        return out.last_hidden_state[0], ids[0], params

    def __call__(self, batch):
        hidden, ids, params = self.hidden_states(batch)
        weight = _head_weight(self.model)
        if not self.calc_log_probs and not self.calc_entropy:
            logits = ops.linear(hidden, weight)
            return pad_input(logits.unsqueeze(0), params)
        # target of token t is token t + 1 of the same packed stream; the roll only mixes
        # sequence ends, which the response window never reads
        target = torch.roll(ids, shifts=-1, dims=0)
        temps = batch.temperatures
        if isinstance(temps, torch.Tensor):
            per_row = (1.0 / temps.to(hidden.device, torch.float32)).reshape(-1, 1).expand(
                -1, batch.input_ids.shape[1])
            inv_t = unpad_input(per_row.unsqueeze(-1).contiguous(), params).reshape(-1)
        elif temps != 1.0:
            inv_t = torch.full((hidden.shape[0],), 1.0 / float(temps), device=hidden.device)
        else:
            inv_t = None
        logp, ent = ops.logprob_entropy(hidden, weight, target, inv_t, ignore_index=self.pad_id)
        r = batch.response_ids.shape[-1]
        logp = pad_input(logp.reshape(1, -1, 1), params).squeeze(-1)[:, -r - 1:-1]
        entropy = None
        if self.calc_entropy:
            entropy = pad_input(ent.reshape(1, -1, 1), params).squeeze(-1)[:, -r - 1:-1]
        return logp, entropy


class ScalarHead(nn.Module):
    def __init__(self, dim, bias=False):
        super().__init__()
        self.linear = nn.Linear(dim, 1, bias=bias)

    def init_weights(self):
        nn.init.normal_(self.linear.weight, std=0.02)
        if self.linear.bias is not None:
            nn.init.zeros_(self.linear.bias)

    def forward(self, hidden):
        return torch.nn.functional.linear(hidden.float(), self.linear.weight.float(),
                                          None if self.linear.bias is None else self.linear.bias.float()
                                          ).squeeze(-1)


class ValueModel(ModelWrapper):
    """Decoder without LM head + scalar head. `__call__(batch)` returns per-token values over
    the response window [B, R] (critic); `score(batch)` the value at the last real token
    (reward model)."""

    def __init__(self, model, value_head: ScalarHead):
        super().__init__(model)
        self.value_head = value_head

    def parameters(self):
        yield from self.model.parameters()
        yield from self.value_head.parameters()

    def _values(self, batch):
        params = build_unpad_params(batch.attention_mask)
        ids = unpad_input(batch.input_ids.unsqueeze(-1), params).squeeze(-1)
        pos = unpad_input(batch.position_ids.unsqueeze(-1), params).squeeze(-1)
        head, self.model.head = getattr(self.model, "head", None), None
        try:
            out = self.model(ids, position_ids=pos, unpad_params=params)
        finally:
            self.model.head = head
        v = self.value_head(out.last_hidden_state[0])
        return pad_input(v.reshape(1, -1, 1), params).squeeze(-1)

    def __call__(self, batch):
        r = batch.response_ids.shape[-1]
        return self._values(batch)[:, -r - 1:-1]

    def score(self, batch):
        v = self._values(batch)
        last = batch.attention_mask.shape[1] - 1 - torch.flip(batch.attention_mask, [1]).argmax(1)
        return v.gather(1, last.unsqueeze(1)).squeeze(1)


class RewardModelScorer:
    """Reward handler backed by a `ValueModel`: called with the `input_ids` and `output_ids`
    columns of a list of rollouts, returns token rewards [n, longest response] that are zero
    except for the model's scalar score at each response's last token."""

    def __init__(self, reward_model: ValueModel, batch_size: int = 16, device=None):
        self.reward_model = reward_model
        self.batch_size = batch_size
        self.device = device

    @torch.no_grad()
    def __call__(self, input_ids, output_ids):
        from halite_b200.projects.common.rollout import Rollout
        from halite_b200.projects.ppo.trainer import build_batch_from_rollouts

        n = len(input_ids)
        longest = max(len(o) for o in output_ids)
        rewards = torch.zeros(n, longest, dtype=torch.float32)
        for lo in range(0, n, self.batch_size):
            hi = min(n, lo + self.batch_size)
            rows = [Rollout(id=str(i), input_ids=input_ids[i], output_ids=output_ids[i], rewards=[0.0])
                    for i in range(lo, hi)]
            batch = build_batch_from_rollouts(rows, device=self.device)
            scores = self.reward_model.score(batch).float().cpu()
            for j, i in enumerate(range(lo, hi)):
                rewards[i, len(output_ids[i]) - 1] = scores[j]
        return rewards
