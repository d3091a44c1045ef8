"""Attention over the paged KV cache: append, prefill (extend) and decode.

CUDA/bf16 runs the hand-written sm_100a kernels (`kv_append`, `paged_prefill`,
`paged_decode` + split merge); the reference path gathers each request's pages into a dense
[seq, heads, dim] tensor and calls the eager attention, and is both the CPU implementation
and the test oracle. Replaces the FlashInfer wrappers and the index_put KV scatter of the
reference (infer/engine/flashinfer_backend.py:126-261, infer/engine/memory_pool.py:139-141).
"""

from __future__ import annotations

import math

import torch

import halite_b200.ops as ops
from halite_b200.ops.attention import attention_reference


def append_kv(k_cache, v_cache, k, v, out_cache_loc):
    """Write new keys / values ([T, Hk, D]) to their flat slots (page * page_size + offset)."""
    if ops.use_sm100(k) and k_cache.dtype == torch.bfloat16:
        kk = k if (k.stride(-1) == 1 and k.stride(-2) == k.shape[-1]) else k.contiguous()
        vv = v if (v.stride(-1) == 1 and v.stride(-2) == v.shape[-1]) else v.contiguous()
        ops.ext().kv_append(k_cache, v_cache, kk, vv, out_cache_loc)
        return
    kc = k_cache.view(-1, *k_cache.shape[2:])
    vc = v_cache.view(-1, *v_cache.shape[2:])
    kc[out_cache_loc] = k.to(kc.dtype)
    vc[out_cache_loc] = v.to(vc.dtype)


def rope_append(q, k, v, k_cache, v_cache, table, out_cache_loc):
    """Fused RoPE + append on the sm_100a path: q [T, Hq, D] is rotated in place (and returned),
    k is rotated while it is written to its page slots, v is copied."""
    def packed(t):
        return t if (t.stride(-1) == 1 and t.stride(-2) == t.shape[-1]) else t.contiguous()

    q, k, v = packed(q), packed(k), packed(v)
    pos = table.positions.reshape(-1)
    if pos.dtype != torch.int64:
        pos = pos.long()
    ops.ext().rope_append(q, k, v, k_cache, v_cache, table.cos, table.sin, pos.contiguous(),
                          out_cache_loc, table.interleaved)
    return q


def gather_request_kv(k_cache, v_cache, page_table_row, seq_len, page_size):
    n_pages = (seq_len + page_size - 1) // page_size
    pages = page_table_row[:n_pages].long()
    k = k_cache[pages].reshape(-1, *k_cache.shape[2:])[:seq_len]
    v = v_cache[pages].reshape(-1, *v_cache.shape[2:])[:seq_len]
    return k, v


def paged_attention_reference(q, k_cache, v_cache, fb, scale=None, softcap=0.0, window=None):
    """q: [T, Hq, D] flat over requests (EXTEND: extend_len tokens each; DECODE: one each)."""
    out = torch.empty_like(q)
    seq_lens = fb.seq_lens_cpu if fb.seq_lens_cpu is not None else fb.seq_lens.tolist()
    if fb.mode.is_decode():
        ext = [1] * len(seq_lens)
    else:
        ext = fb.extend_lens_cpu if fb.extend_lens_cpu is not None else fb.extend_lens.tolist()
    slots = fb.req_slots.tolist()
    start = 0
    for slot, sl, el in zip(slots, seq_lens, ext):
        k, v = gather_request_kv(k_cache, v_cache, fb.page_table[slot], sl, fb.page_size)
        qi = q[start:start + el]
        o = attention_reference(qi[None], k[None], v[None], causal=True, scale=scale, softcap=softcap,
                                window=window, q_offset=None)
        out[start:start + el] = o[0]
        start += el
    return out


def paged_prefill_attention(q, k_cache, v_cache, fb, scale=None, softcap=0.0, window=None):
    if ops.use_sm100(q) and k_cache.dtype == torch.bfloat16 and not softcap and window is None \
            and q.shape[-1] in (64, 128):
        scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
        if not (q.stride(-1) == 1 and q.stride(-2) == q.shape[-1]):
            q = q.contiguous()
        out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        ops.ext().paged_prefill(q, k_cache, v_cache, out, fb.page_table, fb.req_slots, fb.qo_indptr,
                                fb.seq_lens, fb.max_extend_len, float(scale), ops.status_word(q.device))
        return out
    return paged_attention_reference(q, k_cache, v_cache, fb, scale, softcap, window)


def paged_decode_attention(q, k_cache, v_cache, fb, scale=None, softcap=0.0, window=None, workspace=None):
    if ops.use_sm100(q) and k_cache.dtype == torch.bfloat16 and not softcap and window is None \
            and q.shape[-1] in (64, 128):
        scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
        if not (q.stride(-1) == 1 and q.stride(-2) == q.shape[-1]):
            q = q.contiguous()
        out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        ops.ext().paged_decode(q, k_cache, v_cache, out, fb.page_table, fb.req_slots, fb.seq_lens,
                               workspace, float(scale), ops.status_word(q.device))
        return out
    return paged_attention_reference(q, k_cache, v_cache, fb, scale, softcap, window)
