"""Self-attention modules (reference: transformers/attention.py:33-1029).

`SelfAttention` (one fused qkv projection) and `SelfAttentionQKV` (separate q, k, v) wrap an
`Attention` core. State-dict keys are `qkv|q|k|v|out.weight` and
`attention.{q_norm,k_norm}.weight`, as in the reference's checkpoints.

B200 path: when the FSDP layer has laid q, k, v out contiguously in its flat parameter
buffer it hands the module one `[q+k+v, dim]` weight view; the three projections then run as
a single tcgen05 GEMM and RoPE + attention consume the packed output in place.
"""

from __future__ import annotations

import math
from collections.abc import Mapping

import torch
from torch import nn
import torch.nn.functional as F

from halite_b200 import ops
from halite_b200.models.initialize import init_weights
from halite_b200.models.position import RotaryTable, apply_rotary_emb
from halite_b200.models.types import UnpadParams
from halite_b200.ops import attention as attn_ops


def unpad_params(attention_mask):
    """Indices and cumulative lengths of the real tokens of a padded batch."""
    seqlens = attention_mask.sum(-1, dtype=torch.int32)
    indices = torch.nonzero(attention_mask.flatten(), as_tuple=False).flatten()
    max_len = int(seqlens.max())
    cu = F.pad(torch.cumsum(seqlens, 0, dtype=torch.int32), (1, 0))
    return indices, cu, max_len


def build_unpad_params(attention_mask):
    indices, cu, max_len = unpad_params(attention_mask)
    return UnpadParams(cu_seqlens_q=cu, max_length_q=max_len, batch=attention_mask.shape[0],
                       seqlen=attention_mask.shape[1], indices_q=indices)


def unpad_input(input, params: UnpadParams):
    """[B, S, ...] -> [1, total, ...] keeping only real tokens."""
    flat = input.reshape(-1, *input.shape[2:])
    return flat.index_select(0, params.indices_q).unsqueeze(0)


def pad_input(input, params: UnpadParams):
    """[1, total, ...] -> [B, S, ...] with zeros at padding."""
    flat = input.squeeze(0)
    out = flat.new_zeros(params.batch * params.seqlen, *flat.shape[1:])
    out.index_copy_(0, params.indices_q, flat)
    return out.view(params.batch, params.seqlen, *flat.shape[1:])


def _is_plain_rope(fn):
    base = getattr(fn, "func", fn)
    return base is apply_rotary_emb


class Attention(nn.Module):
    """softmax(QK^T * scale [+ bias]) V with GQA, causal / window / document masks, softcap,
    optional q/k norm and a position-embedding hook.

    `processor` names which fused implementation the reference would call ("flash_attn",
    "torch", "flex", "native", "auto"); here every choice ends in the same dispatcher
    (`ops.attention.attention`), "native" forcing the eager fp32 path.
    """

    def __init__(self, n_heads, head_dim, n_key_value_heads=None, attn_drop=0, is_causal=False,
                 apply_pos_emb_fn=None, processor="auto", normalize=True, softcap=0.0, q_norm=None,
                 k_norm=None, window_size=None, **processor_kwargs):
        super().__init__()
        self.n_heads = n_heads
        self.head_dim = head_dim
        self.n_key_value_heads = n_key_value_heads
        self.attn_drop_p = attn_drop
        self.attn_drop = nn.Dropout(attn_drop)
        self.is_causal = is_causal
        self.apply_pos_emb_fn = apply_pos_emb_fn
        self.processor = processor
        self.softcap = softcap
        self.q_norm = q_norm
        self.k_norm = k_norm
        self.window_size = window_size
        self.attention_kwargs = processor_kwargs
        self.normalize = normalize
        if isinstance(normalize, bool):
            self.normalize = 1 / math.sqrt(head_dim) if normalize else 1.0

    @property
    def kv_heads(self):
        return self.n_key_value_heads or self.n_heads

    def forward(self, query, key, value, attention_mask=None, attention_bias=None, pos_embed=None,
                cache=None, use_cache=False, unpad_params=None):
        batch, q_len, _ = query.shape
        k_len = key.shape[1]
        query = query.view(batch, q_len, -1, self.head_dim)
        key = key.view(batch, k_len, -1, self.head_dim)
        value = value.view(batch, k_len, -1, self.head_dim)
        if self.q_norm is not None:
            query = self.q_norm(query)
        if self.k_norm is not None:
            key = self.k_norm(key)
        if self.apply_pos_emb_fn is not None and pos_embed is not None:
            query, key = self.apply_pos_emb_fn(query, key, pos_embed)
        next_cache = None
        if cache is not None:
            if hasattr(cache, "get"):           # cache objects append in their own way
                key, value = cache.get(key, value)
            else:
                key = torch.cat((cache[0], key), 1)
                value = torch.cat((cache[1], value), 1)
        if use_cache:
            next_cache = (key, value)
        out = self.core(query, key, value, attention_mask, attention_bias, unpad_params)
        return out.reshape(batch, q_len, -1), next_cache

    def core(self, query, key, value, attention_mask=None, attention_bias=None, unpad_params=None):
        """[B,S,H,D] tensors -> [B,S,H,D]. `attention_mask` is either a boolean tensor (True =
        blocked), or a mask spec produced by the flex-attention mask classes."""
        kwargs = dict(causal=self.is_causal, scale=self.normalize, softcap=self.softcap,
                      window=self.window_size)
        if unpad_params is not None:
            return attn_ops.attention(query, key, value, cu_seqlens=unpad_params.cu_seqlens_q,
                                      max_seqlen=unpad_params.max_length_q, **kwargs)
        mask = attention_mask
        if mask is not None and hasattr(mask, "to_attention_kwargs"):
            resolved = mask.to_attention_kwargs(query.shape[1], key.shape[1], query.device)
            if resolved.get("window") is None:
                resolved.pop("window", None)         # the module's own window stays in force
            kwargs.update(resolved)
            mask = kwargs.pop("mask", None)
        if self.processor == "native" or attention_bias is not None or mask is not None:
            if mask is not None and mask.dtype != torch.bool:
                # additive float mask
                attention_bias = mask if attention_bias is None else attention_bias + mask
                mask = None
            return attn_ops.attention_reference(query, key, value, mask=mask, bias=attention_bias,
                                                q_offset=None, **kwargs)
        return attn_ops.attention(query, key, value, **kwargs)


class _SelfAttentionBase(nn.Module):
    def _select_layer_type(self, attention_mask, attention_bias, pos_emb):
        if self.layer_type is not None:
            if isinstance(attention_mask, Mapping):
                attention_mask = attention_mask[self.layer_type]
            if isinstance(attention_bias, Mapping):
                attention_bias = attention_bias[self.layer_type]
            if isinstance(pos_emb, Mapping):
                pos_emb = pos_emb[self.layer_type]
        return attention_mask, attention_bias, pos_emb

    def _packed_ok(self, input, attention_mask, attention_bias, pos_emb, cache, use_cache, unpad):
        a = self.attention
        return (type(a) is Attention                     # subclasses (differential attention) have their own core
                and ops.use_sm100(input) and attention_mask is None and attention_bias is None
                and cache is None and not use_cache and unpad is None
                and a.q_norm is None and a.k_norm is None and not a.softcap and a.window_size is None
                and a.processor != "native" and self.scaler is None
                and (pos_emb is None or isinstance(pos_emb, RotaryTable))
                and (a.apply_pos_emb_fn is None or _is_plain_rope(a.apply_pos_emb_fn))
                and not (self.training and a.attn_drop_p > 0))

    def _packed_forward(self, input, weight, bias, pos_emb):
        a = self.attention
        qkv = ops.linear(input, weight, bias)
        if pos_emb is not None and a.apply_pos_emb_fn is not None:
            out = attn_ops.packed_qkv_attention(qkv, a.n_heads, a.kv_heads, a.head_dim, pos_emb.cos,
                                                pos_emb.sin, pos_emb.positions, pos_emb.interleaved,
                                                a.is_causal, a.normalize)
        else:
            out = attn_ops.packed_qkv_attention(qkv, a.n_heads, a.kv_heads, a.head_dim, causal=a.is_causal,
                                                scale=a.normalize)
        return ops.linear(out, self.out.weight, self.out.bias)


def _tp_attention(module, input, pos_emb, qkv_weights):
    """Tensor-parallel attention on a token shard: all-gather fused into the (first) projection,
    attention over this rank's heads, output projection fused with the reduce-scatter."""
    from halite_b200.parallel.tensor_parallel import ag_linear, linear_rs

    tp = module._hb_tp
    B, S = tp.batch_shape
    a = module.attention
    x = input.reshape(-1, input.shape[-1])
    # separate q / k / v parameters that are not contiguous in memory are concatenated so the
    # gathered input feeds one GEMM and its gradient flows back through one reduce-scatter
    w = qkv_weights[0] if len(qkv_weights) == 1 else torch.cat(list(qkv_weights), 0)
    qkv, _ = ag_linear(x, w, tp)
    qkv = qkv.view(B, S, -1)
    if pos_emb is not None and a.apply_pos_emb_fn is not None:
        out = attn_ops.packed_qkv_attention(qkv, a.n_heads, a.kv_heads, a.head_dim, pos_emb.cos, pos_emb.sin,
                                            pos_emb.positions, pos_emb.interleaved, a.is_causal, a.normalize)
    else:
        out = attn_ops.packed_qkv_attention(qkv, a.n_heads, a.kv_heads, a.head_dim, causal=a.is_causal,
                                            scale=a.normalize)
    out = linear_rs(out.reshape(B * S, -1), module.out.weight, tp)
    return out.view(1, -1, out.shape[-1])


class SelfAttention(_SelfAttentionBase):
    """Fused qkv projection. `qkv_split="llama"`: rows are [q | k | v]; `"megatron"`: rows are
    grouped per KV head as [q_group, k, v]."""

    def __init__(self, qkv, attention, out, qkv_split="llama", qkv_init=None, out_init=None,
                 scaler=None, layer_type=None):
        super().__init__()
        self.qkv = qkv
        self.attention = attention
        self.out = out
        self.qkv_split = qkv_split
        self.qkv_init = qkv_init
        self.out_init = out_init
        self.scaler = scaler
        self.layer_type = layer_type
        self.n_heads = attention.n_heads
        self.head_dim = attention.head_dim
        self.n_key_value_heads = attention.n_key_value_heads or attention.n_heads

    def init_weights(self):
        init_weights(self.qkv, self.qkv_init)
        init_weights(self.out, self.out_init)

    def split(self, qkv):
        H, Hk, D = self.n_heads, self.n_key_value_heads, self.head_dim
        if self.qkv_split == "megatron":
            g = H // Hk
            x = qkv.unflatten(-1, (Hk, g + 2, D))
            q = x[..., :g, :].flatten(-3)
            k = x[..., g, :].flatten(-2)
            v = x[..., g + 1, :].flatten(-2)
            return q, k, v
        return qkv.split((H * D, Hk * D, Hk * D), -1)

    def forward(self, input, attention_mask=None, attention_bias=None, pos_emb=None, cache=None,
                use_cache=False, unpad_params=None):
        attention_mask, attention_bias, pos_emb = self._select_layer_type(attention_mask, attention_bias, pos_emb)
        if getattr(self, "_hb_tp", None) is not None:
            return _tp_attention(self, input, pos_emb, [self.qkv.weight]), None
        if self.qkv_split == "llama" and self._packed_ok(input, attention_mask, attention_bias, pos_emb,
                                                         cache, use_cache, unpad_params):
            return self._packed_forward(input, self.qkv.weight, self.qkv.bias, pos_emb), None
        qkv = ops.linear(input, self.qkv.weight, self.qkv.bias)
        q, k, v = self.split(qkv)
        if self.scaler is not None:
            q, k = self.scaler(q), self.scaler(k)
        out, next_cache = self.attention(q, k, v, attention_mask, attention_bias, pos_emb, cache,
                                         use_cache, unpad_params=unpad_params)
        return ops.linear(out, self.out.weight, self.out.bias), next_cache

    def tp_plan(self):
        return {"qkv": "colwise_qkv", "out": "rowwise"}


class SelfAttentionQKV(_SelfAttentionBase):
    def __init__(self, q, k, v, attention, out, q_init=None, k_init=None, v_init=None, out_init=None,
                 scaler=None, q_norm=None, k_norm=None, layer_type=None):
        super().__init__()
        self.q, self.k, self.v = q, k, v
        self.attention = attention
        self.out = out
        self.scaler = scaler
        self.n_heads = attention.n_heads
        self.head_dim = attention.head_dim
        self.n_key_value_heads = attention.n_key_value_heads or attention.n_heads
        self.q_init, self.k_init, self.v_init, self.out_init = q_init, k_init, v_init, out_init
        self.q_norm, self.k_norm = q_norm, k_norm
        self.layer_type = layer_type

    def init_weights(self):
        init_weights(self.q, self.q_init)
        init_weights(self.k, self.k_init)
        init_weights(self.v, self.v_init)
        init_weights(self.out, self.out_init)

    def fusable_linears(self):
        """Groups of linears that read the same input: laid out contiguously they run as one GEMM."""
        return {"qkv": ("q", "k", "v")}

    def forward(self, input, attention_mask=None, attention_bias=None, pos_emb=None, cache=None,
                use_cache=False, unpad_params=None):
        attention_mask, attention_bias, pos_emb = self._select_layer_type(attention_mask, attention_bias, pos_emb)
        fused = getattr(self, "_hb_fused", {}).get("qkv")
        if getattr(self, "_hb_tp", None) is not None:
            ws = [fused] if fused is not None else [self.q.weight, self.k.weight, self.v.weight]
            return _tp_attention(self, input, pos_emb, ws), None
        if fused is not None and self.q_norm is None and self.k_norm is None and \
                self._packed_ok(input, attention_mask, attention_bias, pos_emb, cache, use_cache, unpad_params):
            return self._packed_forward(input, fused, None, pos_emb), None
        if fused is not None and ops.use_sm100(input):
            q, k, v = ops.linear(input, fused).split(
                (self.q.weight.shape[0], self.k.weight.shape[0], self.v.weight.shape[0]), -1)
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
        out, next_cache = self.attention(q, k, v, attention_mask, attention_bias, pos_emb, cache,
                                         use_cache, unpad_params=unpad_params)
        return ops.linear(out, self.out.weight, self.out.bias), next_cache

    def tp_plan(self):
        return {"q": "colwise", "k": "colwise", "v": "colwise", "out": "rowwise"}


class DiffAttention(Attention):
    """Differential attention: two softmax maps from split heads, subtracted with a learned
    lambda, followed by a per-head norm scaled by (1 - lambda_init)."""

    def __init__(self, n_heads, head_dim, lambda_init=None, n_key_value_heads=None, is_causal=True,
                 apply_pos_emb_fn=None, sub_norm=None, layer_id=None, **kwargs):
        super().__init__(n_heads, head_dim, n_key_value_heads, is_causal=is_causal,
                         apply_pos_emb_fn=apply_pos_emb_fn, **kwargs)
        if lambda_init is None:      # the schedule of the paper, by depth
            lambda_init = 0.8 - 0.6 * math.exp(-0.3 * (layer_id or 0))
        self.lambda_init = lambda_init
        self.lambda_q1 = nn.Parameter(torch.zeros(head_dim))
        self.lambda_k1 = nn.Parameter(torch.zeros(head_dim))
        self.lambda_q2 = nn.Parameter(torch.zeros(head_dim))
        self.lambda_k2 = nn.Parameter(torch.zeros(head_dim))
        self.sub_norm = sub_norm

    def init_weights(self):
        for p in (self.lambda_q1, self.lambda_k1, self.lambda_q2, self.lambda_k2):
            nn.init.normal_(p, mean=0, std=0.1)

    def core(self, query, key, value, attention_mask=None, attention_bias=None, unpad_params=None):
        # heads come in pairs (2h, 2h+1) for q and k; v heads carry 2 * head_dim
        B, S, H2, D = query.shape
        q1, q2 = query[:, :, 0::2], query[:, :, 1::2]
        k1, k2 = key[:, :, 0::2], key[:, :, 1::2]
        v = value.reshape(B, value.shape[1], -1, 2 * D)
        a1 = super().core(q1, k1, v, attention_mask, attention_bias, unpad_params)
        a2 = super().core(q2, k2, v, attention_mask, attention_bias, unpad_params)
        lam1 = torch.exp(torch.sum(self.lambda_q1 * self.lambda_k1, -1).float())
        lam2 = torch.exp(torch.sum(self.lambda_q2 * self.lambda_k2, -1).float())
        lam = (lam1 - lam2 + self.lambda_init).to(a1.dtype)
        out = a1 - lam * a2
        if self.sub_norm is not None:
            out = self.sub_norm(out)
        out = out * (1 - self.lambda_init)
        return out.reshape(B, S, H2, D)
