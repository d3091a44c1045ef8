// Host entry points of the sm_100a training attention kernels (no torch headers).
//
// Self-attention over a flat token space: `total` tokens, each belonging to one segment (a
// sequence of a [batch, seq] tensor, a document of a packed batch). Token q may attend token k
// when both lie in the same segment and
//     causal:      k <= q            (else k anywhere in the segment)
//     window > 0:  q - k < window    (how far back a query looks; keys after q are not limited)
// Segments are either equal-length (`seq_len`, token t belongs to segment t / seq_len) or given
// per token by `seg_start[t]` / `seg_end[t]` (first token of t's segment, one past its last):
// that one form covers fixed batches, `cu_seqlens` packing and document masks, and keeps every
// length on the device.
//
// Layouts (bf16 unless noted): q [total, n_heads, head_dim] with `q_tok_stride` elements between
// tokens (heads adjacent, so slices of a packed qkv projection work), k / v likewise with
// n_kv_heads (n_heads % n_kv_heads == 0: grouped-query attention), out [total, n_heads,
// head_dim] contiguous, lse fp32 [n_heads, total] (natural log of the softmax denominator).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

// #define HB_ATTN_PROFILE 1   // cycle counters of the backward kernel (see attention_sm100.cu)

namespace hb {

#ifdef HB_ATTN_PROFILE
// 32 cycle counters of the backward kernel's roles, summed over CTAs since the last reset.
cudaError_t attention_profile_read(unsigned long long* out32, bool reset);
#endif

struct AttnArgs {
  const void* q = nullptr;
  const void* k = nullptr;
  const void* v = nullptr;
  long q_tok_stride = 0, k_tok_stride = 0, v_tok_stride = 0;   // elements
  int total = 0;
  int n_heads = 0, n_kv_heads = 0, head_dim = 0;   // head_dim 64 or 128
  int seq_len = 0;                 // used when seg_start == nullptr
  const int* seg_start = nullptr;  // [total] or nullptr
  const int* seg_end = nullptr;    // [total] or nullptr
  bool causal = true;
  int window = 0;                  // <= 0: no window
  float scale = 1.f;
  float softcap = 0.f;             // > 0: scores become softcap * tanh(score / softcap)
  int* status = nullptr;           // device int set to a WaitCode when a bounded wait gave up
  cudaStream_t stream = nullptr;
};

// out = softmax(mask(scale * q k^T)) v, plus the log-sum-exp per (head, token).
cudaError_t attention_fwd(const AttnArgs& a, void* out, float* lse);

// Optional inverse rotation of dQ on its way out (q was rotated in place before the forward):
// cos / sin fp32 [max_position, rot_dim / 2], one position per token. cos == nullptr: none.
struct AttnDqRotation {
  const float* cos = nullptr;
  const float* sin = nullptr;
  const void* positions = nullptr;
  bool pos_is_i64 = true;
  int rot_dim = 0;
  bool interleaved = true;
};

// Gradients. `o`, `d_o`: [total, n_heads, head_dim] contiguous bf16; `lse` from the forward.
// `delta` fp32 [n_heads, total] and `dq_accum` fp32 [total, n_heads, head_dim] are scratch the
// caller provides (dq_accum is zeroed here). dq: bf16 [total, n_heads, head_dim] and dk, dv:
// bf16 [total, n_kv_heads, head_dim], each with its own number of elements between tokens, so
// all three may be slots of one packed qkv gradient.
cudaError_t attention_bwd(const AttnArgs& a, const void* o, const void* d_o, const float* lse,
                          float* delta, float* dq_accum, void* dq, long dq_tok_stride,
                          const AttnDqRotation& rot, void* dk, long dk_tok_stride, void* dv,
                          long dv_tok_stride);

}  // namespace hb
