"""Positional encodings (reference: transformers/position.py:10-388): rotary embeddings with
plain, linearly scaled and Llama-3 scaled frequencies, ALiBi, learned positions.

A rotary module returns a `RotaryTable` (fp32 cos/sin tables + the positions to read); the
rotation itself is `apply_rotary_emb`, which runs the sm_100a kernel on CUDA/bf16 and the
eager formula elsewhere. `use_complex` and the default matrix mode rotate interleaved pairs
(x[2i], x[2i+1]); `use_rotate_half` / `use_fused` rotate (x[i], x[i + d/2]).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import nn

from halite_b200 import ops
from halite_b200.ops.rope import llama3_scale_inv_freq, rope_tables


@dataclass
class RotaryTable:
    cos: torch.Tensor          # [max_pos, dim/2] fp32
    sin: torch.Tensor
    positions: torch.Tensor    # integer positions, broadcastable to the token dims
    interleaved: bool
    unpad_params: object | None = None


def make_causal_mask(batch_size, query_length, key_length, device):
    """Boolean mask, True where attention is not allowed; None for single-token queries."""
    if query_length <= 1:
        return None
    mask = torch.ones((query_length, key_length), dtype=torch.bool, device=device)
    mask = torch.triu(mask, key_length - query_length + 1)
    return mask.expand(batch_size, 1, query_length, key_length)


class RotaryEmbedding(nn.Module):
    attention_bias = False
    layer_shared = True

    def __init__(self, dim, max_position_embeddings=2048, base=10000, device=None, use_complex=False,
                 use_rotate_half=False, use_fused=False, pre_init=False, use_fp32=False):
        super().__init__()
        self.dim = dim
        self.max_position_embeddings = max_position_embeddings
        self.base = base
        self.use_complex = use_complex
        self.use_rotate_half = use_rotate_half
        self.use_fused = use_fused
        self.pre_init = pre_init
        self.use_fp32 = use_fp32
        self._cos = self._sin = None
        self._cached = 0
        self.init_buffers(device)

    @property
    def interleaved(self):
        return not (self.use_rotate_half or self.use_fused)

    def get_inv_freq(self):
        # explicit CPU device: models are often constructed under `torch.device("meta")`
        return 1.0 / (self.base ** (torch.arange(0, self.dim, 2, dtype=torch.float32, device="cpu") / self.dim))

    def init_buffers(self, device=None):
        self.inv_freq = self.get_inv_freq()
        self._cached = 0
        self._cos = self._sin = None
        if self.pre_init and device is not None and torch.device(device).type != "meta":
            self._grow(self.max_position_embeddings, device)

    def _grow(self, seq_len, device):
        # tables are built on the host in fp32 so every device sees identical values
        seq_len = max(int(seq_len), self.max_position_embeddings)
        cos, sin = rope_tables(self.inv_freq.cpu(), seq_len)
        self._cos, self._sin = cos.to(device), sin.to(device)
        self._cached = seq_len

    def tables(self, seq_len, device):
        if self._cos is None or seq_len > self._cached or self._cos.device != torch.device(device):
            self._grow(max(seq_len, self._cached), device)
        return self._cos, self._sin

    def forward(self, position_ids, seq_len=None, unpad_params=None, device=None, dtype=None):
        if device is None:
            device = position_ids.device
        cos, sin = self.tables(max(seq_len or 0, self.max_position_embeddings), device)
        if position_ids is None:
            position_ids = torch.arange(seq_len, device=device).unsqueeze(0)
        return RotaryTable(cos, sin, position_ids, self.interleaved, unpad_params)


class LinearRoPE(RotaryEmbedding):
    def __init__(self, dim, max_position_embeddings, base=10000, device=None, use_complex=False,
                 use_rotate_half=False, scaling=1.0):
        self.scaling = scaling
        super().__init__(dim, max_position_embeddings, base, device, use_complex, use_rotate_half)

    def get_inv_freq(self):
        return super().get_inv_freq() / self.scaling


class Llama3RoPE(RotaryEmbedding):
    def __init__(self, dim, max_position_embeddings=8192, base=500000, use_scaled_rope=False,
                 scale_factor=8, low_freq_factor=1, high_freq_factor=4, original_context_len=8192,
                 device=None, use_complex=False):
        self.use_scaled_rope = use_scaled_rope
        self.scale_factor = scale_factor
        self.low_freq_factor = low_freq_factor
        self.high_freq_factor = high_freq_factor
        self.original_context_len = original_context_len
        super().__init__(dim, max_position_embeddings, base, device, use_complex)

    def get_inv_freq(self):
        inv_freq = super().get_inv_freq()
        if self.use_scaled_rope:
            inv_freq = llama3_scale_inv_freq(inv_freq, self.scale_factor, self.low_freq_factor,
                                             self.high_freq_factor, self.original_context_len)
        return inv_freq


def apply_rotary_emb(query, key, pos_embed, use_fp32=False, use_complex=False, use_fused=False,
                     inplace=False):
    """Rotate query / key ([..., heads, head_dim]) by a `RotaryTable`."""
    if pos_embed is None:
        return query, key
    return ops.apply_rope(query, key, pos_embed.cos, pos_embed.sin, pos_embed.positions,
                          pos_embed.interleaved)


def alibi_slopes(n_heads, device=None):
    closest = 2 ** math.floor(math.log2(n_heads))
    base = 2.0 ** (-(2.0 ** -(math.log2(closest) - 3)))
    slopes = torch.pow(torch.tensor(base, dtype=torch.float32), torch.arange(1, 1 + closest))
    if closest != n_heads:
        extra_base = 2.0 ** (-(2.0 ** -(math.log2(2 * closest) - 3)))
        n_rem = min(closest, n_heads - closest)
        extra = torch.pow(torch.tensor(extra_base, dtype=torch.float32), torch.arange(1, 1 + 2 * n_rem, 2))
        slopes = torch.cat((slopes, extra), 0)
    return slopes.to(device) if device is not None else slopes


class ALiBi(nn.Module):
    """Linear attention bias: slope_h * key_position (softmax is shift invariant per row)."""

    attention_bias = True
    layer_shared = True

    def __init__(self, n_heads, attention_mask=None, device=None):
        super().__init__()
        self.n_heads = n_heads
        self.register_buffer("slopes", alibi_slopes(n_heads), persistent=False)

    def forward(self, attention_mask):
        # attention_mask: [batch, key_length] with 1 for real tokens
        pos = (attention_mask.to(torch.float32).cumsum(-1) - 1).clamp(min=0) * attention_mask
        return self.slopes.view(1, -1, 1, 1).to(pos.device) * pos[:, None, None, :]


class LearnedPositionEmbedding(nn.Module):
    def __init__(self, dim, max_position_embeddings):
        super().__init__()
        self.pos_embed = nn.Parameter(torch.zeros(max_position_embeddings, dim))

    def init_weights(self):
        nn.init.normal_(self.pos_embed, std=0.02)

    def forward(self, input):
        return input + self.pos_embed[: input.shape[1]].unsqueeze(0)
