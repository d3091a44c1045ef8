"""Inference-time attention modules (reference: infer/attention.py:10-228): the projections of
the training modules with a paged-KV attention core. Activations are flat: [tokens, dim].

`pack_weights()` lays q|k|v (and up|gate in the feed-forward) out as one matrix so each
group of projections is a single GEMM; the separate parameters become views of it and the
state-dict keys stay those of the training model.
"""

from __future__ import annotations

import math

import torch
from torch import nn

from halite_b200 import ops
from halite_b200.models.initialize import init_weights
from halite_b200.models.position import RotaryTable, apply_rotary_emb
from halite_b200.ops import paged_attention as pa
from halite_b200.infer.tensor_parallel import row_parallel_linear


def _is_plain_rope(fn):
    return getattr(fn, "func", fn) is apply_rotary_emb


class PagedAttention(nn.Module):
    def __init__(self, layer_id, n_heads, head_dim, n_key_value_heads=None, apply_pos_emb_fn=None,
                 normalize=True, q_norm=None, k_norm=None, softcap=0.0, window_size=None):
        super().__init__()
        self.layer_id = layer_id
        self.n_heads = n_heads
        self.head_dim = head_dim
        self.n_key_value_heads = n_key_value_heads
        self.apply_pos_emb_fn = apply_pos_emb_fn
        self.q_norm = q_norm
        self.k_norm = k_norm
        self.softcap = softcap or 0.0
        self.window_size = window_size
        self.normalize = normalize
        if isinstance(normalize, bool):
            self.normalize = 1 / math.sqrt(head_dim) if normalize else 1.0
        self.kv_pool = None       # set by the model runner

    @property
    def kv_heads(self):
        return self.n_key_value_heads or self.n_heads

    def forward(self, query, key, value, forward_batch, pos_embed=None):
        T = query.shape[0]
        q = query.view(T, -1, self.head_dim)
        k = key.view(T, -1, self.head_dim)
        v = value.view(T, -1, self.head_dim)
        if self.q_norm is not None:
            q = self.q_norm(q)
        if self.k_norm is not None:
            k = self.k_norm(k)
        k_cache, v_cache = self.kv_pool.get_kv_buffer(self.layer_id)
        rope = self.apply_pos_emb_fn is not None and pos_embed is not None
        if rope and isinstance(pos_embed, RotaryTable) and _is_plain_rope(self.apply_pos_emb_fn) \
                and ops.use_sm100(q) and k_cache.dtype == torch.bfloat16:
            # one kernel: rotate q in place, rotate k on its way into the pages, copy v
            q = pa.rope_append(q, k, v, k_cache, v_cache, pos_embed, forward_batch.out_cache_loc)
        else:
            if rope:
                q, k = self.apply_pos_emb_fn(q, k, pos_embed)
            pa.append_kv(k_cache, v_cache, k, v, forward_batch.out_cache_loc)
        if forward_batch.mode.is_decode():
            out = pa.paged_decode_attention(q, k_cache, v_cache, forward_batch, self.normalize,
                                            self.softcap, self.window_size,
                                            getattr(forward_batch, "workspace", None))
        else:
            out = pa.paged_prefill_attention(q, k_cache, v_cache, forward_batch, self.normalize,
                                             self.softcap, self.window_size)
        return out.reshape(T, -1)


def _pack(linears):
    """Concatenate linear weights row-wise into one buffer; the originals become views."""
    ws = [l.weight for l in linears]
    if any(getattr(l, "bias", None) is not None for l in linears) or ws[0].device.type == "meta":
        return None
    packed = torch.cat([w.detach() for w in ws], 0).contiguous()
    row = 0
    for l in linears:
        n = l.weight.shape[0]
        l.weight = nn.Parameter(packed[row:row + n], requires_grad=False)
        row += n
    return packed


class InferSelfAttentionQKV(nn.Module):
    def __init__(self, q, k, v, attention, out, q_init=None, k_init=None, v_init=None, out_init=None,
                 scaler=None, q_norm=None, k_norm=None, layer_type=None):
        super().__init__()
        self.q, self.k, self.v = q, k, v
        self.attention = attention
        self.out = out
        self.q_init, self.k_init, self.v_init, self.out_init = q_init, k_init, v_init, out_init
        self.scaler = scaler
        self.q_norm, self.k_norm = q_norm, k_norm
        self.layer_type = layer_type
        self._packed = None

    def init_weights(self):
        init_weights(self.q, self.q_init)
        init_weights(self.k, self.k_init)
        init_weights(self.v, self.v_init)
        init_weights(self.out, self.out_init)
        self._packed = None

    def pack_weights(self):
        self._packed = _pack([self.q, self.k, self.v])

    def forward(self, input, forward_batch, pos_emb=None):
        if self._packed is not None:
            qkv = ops.linear(input, self._packed)
            q, k, v = qkv.split((self.q.weight.shape[0], self.k.weight.shape[0], self.v.weight.shape[0]), -1)
        else:
            q = ops.linear(input, self.q.weight, self.q.bias)
            k = ops.linear(input, self.k.weight, self.k.bias)
            v = ops.linear(input, self.v.weight, self.v.bias)
        if self.q_norm is not None:
            q = self.q_norm(q)
        if self.k_norm is not None:
            k = self.k_norm(k)
        if self.scaler is not None:
            q, k = self.scaler(q), self.scaler(k)
        if self.layer_type is not None and isinstance(pos_emb, dict):
            pos_emb = pos_emb[self.layer_type]
        out = self.attention(q, k, v, forward_batch, pos_emb)
        return row_parallel_linear(self, out, self.out)


class InferSelfAttention(nn.Module):
    def __init__(self, qkv, attention, out, qkv_split="llama", qkv_init=None, out_init=None, scaler=None,
                 layer_type=None):
        super().__init__()
        self.qkv = qkv
        self.attention = attention
        self.out = out
        self.qkv_split = qkv_split
        self.qkv_init, self.out_init = qkv_init, out_init
        self.scaler = scaler
        self.layer_type = layer_type

    def init_weights(self):
        init_weights(self.qkv, self.qkv_init)
        init_weights(self.out, self.out_init)

    def pack_weights(self):
        pass

    def forward(self, input, forward_batch, pos_emb=None):
        a = self.attention
        H, Hk, D = a.n_heads, a.kv_heads, a.head_dim
        qkv = ops.linear(input, self.qkv.weight, self.qkv.bias)
        if self.qkv_split == "megatron":
            g = H // Hk
            x = qkv.unflatten(-1, (Hk, g + 2, D))
            q, k, v = x[..., :g, :].flatten(-3), x[..., g, :].flatten(-2), x[..., g + 1, :].flatten(-2)
        else:
            q, k, v = qkv.split((H * D, Hk * D, Hk * D), -1)
        if self.scaler is not None:
            q, k = self.scaler(q), self.scaler(k)
        if self.layer_type is not None and isinstance(pos_emb, dict):
            pos_emb = pos_emb[self.layer_type]
        out = a(q, k, v, forward_batch, pos_emb)
        return row_parallel_linear(self, out, self.out)
