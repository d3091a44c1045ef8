"""Small helpers for the expert layers (reference: transformers/moe/ops.py)."""

import torch


def bincount(x: torch.Tensor, minlength: int) -> torch.Tensor:
    """Deterministic per-expert token counts ([minlength] int64). Values >= minlength (the marker
    of a dropped slot) are not counted."""
    x = x.reshape(-1)
    x = x[x < minlength]
    return torch.zeros(minlength, dtype=torch.long, device=x.device).scatter_add_(0, x, torch.ones_like(x))
