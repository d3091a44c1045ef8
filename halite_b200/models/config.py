"""Architecture summary stored next to checkpoints (reference: transformers/config.py:4-14)."""

from __future__ import annotations

from pydantic import BaseModel, ConfigDict


class TransformerConfig(BaseModel):
    model_config = ConfigDict(extra="allow", protected_namespaces=())

    vocab_size: int | None = None
    dim: int | None = None
    n_layers: int | None = None
    n_heads: int | None = None
    head_dim: int | None = None
    n_key_value_heads: int | None = None
    intermediate_size: int | None = None
    context_len: int | None = None
