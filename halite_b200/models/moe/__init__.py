"""Mixture-of-experts layers (reference: transformers/moe/*)."""

from .experts import ExpertLinear, FeedForward, expert_boundaries, grouped_matmul
from .moe import MoE
from .router import TopKRouter, get_capacity, top_k_softmax_with_capacity
from .token_dispatcher import AlltoAllTokenDispatcher

__all__ = ["ExpertLinear", "FeedForward", "expert_boundaries", "grouped_matmul", "MoE", "TopKRouter",
           "get_capacity", "top_k_softmax_with_capacity", "AlltoAllTokenDispatcher"]
