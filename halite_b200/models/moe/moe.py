"""MoE layer: router -> (optional expert-parallel dispatch) -> experts -> combine
(reference: transformers/moe/moe.py:4-31; there the dispatched branch never calls the experts,
here it does)."""

from torch import nn


class MoE(nn.Module):
    def __init__(self, router, token_dispatcher, experts):
        super().__init__()
        self.router, self.token_dispatcher, self.experts = router, token_dispatcher, experts

    def parallelize(self, ep_group):
        self.token_dispatcher.parallelize(ep_group)

    def forward(self, inputs):
        probs, indices, aux_losses = self.router(inputs)
        if self.token_dispatcher is None or not getattr(self.token_dispatcher, "active", False):
            return self.experts(inputs, probs, indices), aux_losses
        return self.token_dispatcher(inputs, probs, indices, self.experts), aux_losses
