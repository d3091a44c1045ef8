// Inference kernels for sm_100a: fused RoPE + KV append into pages, paged decode attention
// (split-KV flash decoding + merge), paged prefill attention (tensor-core tiles, causal with a
// cached-prefix offset) and single-pass Gumbel-max sampling.
//
// KV cache layout per layer: K and V are [pages, page_size = 16, kv_heads, head_dim] bf16; a
// token's flat slot is page * 16 + offset. The page table is [request slots, max pages] int32.
// These replace the FlashInfer wrappers, the Triton index kernel and the index_put scatter
// of the reference engine (infer/engine/flashinfer_backend.py:15-261, memory_pool.py:139-141,
// sampler.py:38-52).
#include <cuda_bf16.h>
#include <math.h>
#include <stdint.h>

#include "infer_kernels.h"

namespace hb {

namespace {

constexpr int kPage = 16;

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ------------------------------------------------------------------ RoPE + append
// One CTA per token. Threads walk (head, pair) items: q is rotated in place, k is rotated on
// its way into the cache, v is copied. cos/sin: [max_pos, rot/2] fp32.
__global__ void rope_append_kernel(__nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                   const __nv_bfloat16* __restrict__ v,
                                   __nv_bfloat16* __restrict__ k_cache,
                                   __nv_bfloat16* __restrict__ v_cache,
                                   const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                   const int64_t* __restrict__ positions,
                                   const int64_t* __restrict__ out_loc, int hq, int hk, int dim,
                                   int rot, long q_stride, long k_stride, long v_stride,
                                   int interleaved, long cache_slots) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // a dependent launch may set itself up under this kernel
  const long t = blockIdx.x;
  const long slot = out_loc[t];
  const bool slot_ok = slot >= 0 && slot < cache_slots;
  const int half = rot >> 1;
  const float* c = cos_t ? cos_t + positions[t] * half : nullptr;
  const float* s = sin_t ? sin_t + positions[t] * half : nullptr;
  __nv_bfloat16* qt = q + t * q_stride;
  const __nv_bfloat16* kt = k + t * k_stride;
  const __nv_bfloat16* vt = v + t * v_stride;
  __nv_bfloat16* kc = k_cache + slot * static_cast<long>(hk) * dim;
  __nv_bfloat16* vc = v_cache + slot * static_cast<long>(hk) * dim;
  const int pairs = dim >> 1;  // items per head: one (even, odd) or (i, i + half) pair
  const int total = (hq + hk) * pairs;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int head = i / pairs;
    const int p = i - head * pairs;
    const bool is_q = head < hq;
    const __nv_bfloat16* src = is_q ? qt + head * dim : kt + (head - hq) * dim;
    int i0, i1;
    float cs = 1.f, sn = 0.f;
    if (p < half && c) {
      if (interleaved) { i0 = 2 * p; i1 = 2 * p + 1; } else { i0 = p; i1 = p + half; }
      cs = c[p];
      sn = s[p];
    } else if (p < half) {
      if (interleaved) { i0 = 2 * p; i1 = 2 * p + 1; } else { i0 = p; i1 = p + half; }
    } else {
      // beyond the rotated span: plain copy of two trailing elements
      i0 = rot + 2 * (p - half);
      i1 = i0 + 1;
    }
    const float a = __bfloat162float(src[i0]);
    const float b = __bfloat162float(src[i1]);
    const __nv_bfloat16 r0 = __float2bfloat16_rn(a * cs - b * sn);
    const __nv_bfloat16 r1 = __float2bfloat16_rn(a * sn + b * cs);
    if (is_q) {
      qt[head * dim + i0] = r0;
      qt[head * dim + i1] = r1;
    } else if (slot_ok) {
      kc[(head - hq) * dim + i0] = r0;
      kc[(head - hq) * dim + i1] = r1;
    }
  }
  if (slot_ok) {
    const int nv = hk * dim / 8;
    for (int i = threadIdx.x; i < nv; i += blockDim.x)
      reinterpret_cast<uint4*>(vc)[i] = reinterpret_cast<const uint4*>(vt)[i];
  }
}

// ------------------------------------------------------------------ decode attention
// grid (batch, kv_heads, splits), 128 threads. A CTA covers tokens [split * chunk, ...) of one
// request for one KV head and all G = hq / hk query heads of its group, in tiles of 64 tokens.
// K and V tiles stream through a three-stage shared-memory ring filled by cp.async, so the loads
// of tiles i+1 and i+2 are in flight while tile i is consumed (decode is bandwidth-bound: what matters is
// bytes in flight, not arithmetic). Rows are padded by 16 bytes so that a warp's 16-byte reads of
// 32 consecutive rows hit distinct banks.
__device__ __forceinline__ void cp_async_16_zfill(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;       // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group_n() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int D>
struct DecodeSmem {
  static constexpr int kTile = 64;
  static constexpr int kRow = D + 8;                       // padded row, elements
  static constexpr int kStages = 3;                        // two tiles in flight while one is consumed
  static constexpr int kStageElems = 2 * kTile * kRow;     // K tile then V tile
  static constexpr int kBytes = kStages * kStageElems * 2; // bf16
};

constexpr int kDecodeThreads = 256;
constexpr int kBadPageId = 8;      // status code: a page table entry named a page outside the pool

template <int D, int G>
__global__ void __launch_bounds__(kDecodeThreads)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                    const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ page_table,
                    const int* __restrict__ req_slots, const int* __restrict__ seq_lens,
                    float* __restrict__ ws, __nv_bfloat16* __restrict__ out, int hq, int hk,
                    int max_pages, int splits, long q_stride, float scale_log2, long num_pages,
                    int* __restrict__ status) {
  using S = DecodeSmem<D>;
  constexpr int TILE = S::kTile;
  constexpr int ROW = S::kRow;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // a dependent launch may set itself up under this kernel
  extern __shared__ __align__(16) unsigned char decode_smem_raw[];
  __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(decode_smem_raw);
  constexpr int NT = kDecodeThreads;
  constexpr int NPART = NT / TILE;          // threads per token in the score phase
  constexpr int NTG = NT / 16;              // token groups in the PV phase
  constexpr int TPG = TILE / NTG;           // tokens per group
  __shared__ float s_scores[G][TILE];
  __shared__ float s_part[NPART][G][TILE];
  __shared__ __align__(16) float s_q[G][D];
  __shared__ float s_alpha[G];
  __shared__ float s_m[G], s_l[G];       // running max / sum when there are more heads than warps
  // the cross-thread reduction at the end reuses the ring (no tile is live by then)
  float (*s_red)[G][D + 1] = reinterpret_cast<float (*)[G][D + 1]>(decode_smem_raw);
  static_assert(sizeof(float) * NTG * G * (D + 1) <= S::kBytes, "reduction scratch must fit in the ring");

  const int b = blockIdx.x, kh = blockIdx.y, sp = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int seq = seq_lens[b];
  const int chunk = ((seq + splits - 1) / splits + TILE - 1) / TILE * TILE;
  const int start = sp * chunk;
  const int end = min(seq, start + chunk);
  const int* pt = page_table + static_cast<long>(req_slots[b]) * max_pages;

  // queries of the group, pre-scaled, in shared memory (read as broadcasts in the dot loop)
  for (int i = tid; i < G * D; i += NT)
    s_q[i / D][i % D] = __bfloat162float(q[b * q_stride + (kh * G + i / D) * D + i % D]) * scale_log2;

  // fill one stage: 64 rows x D elements of K and of V, 16 bytes per copy
  auto load_tile = [&](int stage, int t0) {
    __nv_bfloat16* sk = ring + stage * S::kStageElems;
    __nv_bfloat16* sv = sk + TILE * ROW;
    constexpr int CH = D / 8;                               // 16-byte chunks per row
    for (int i = tid; i < TILE * CH; i += NT) {
      const int row = i / CH, ch = i - row * CH;
      const int t = t0 + row;
      const bool valid = t < end;
      long slot = 0;
      if (valid) {
        const int pi = t >> 4;
        int pg = pi < max_pages ? pt[pi] : -1;
        if (pg < 0 || pg >= num_pages) {
          // a page id outside the pool: read the scratch page (the access stays in bounds) and
          // report it through the status word, the way every bounded wait reports a failure
          if (status) atomicCAS(status, 0, kBadPageId);
          pg = 0;
        }
        slot = static_cast<long>(pg) * kPage + (t & 15);
      }
      const long off = (slot * hk + kh) * D + ch * 8;
      cp_async_16_zfill(static_cast<uint32_t>(__cvta_generic_to_shared(sk + row * ROW + ch * 8)), k_cache + off, valid);
      cp_async_16_zfill(static_cast<uint32_t>(__cvta_generic_to_shared(sv + row * ROW + ch * 8)), v_cache + off, valid);
    }
    cp_async_commit_group();
  };

  // QK mapping: thread -> (token = tid % 64, slice of the head dim = tid / 64): a warp reads 32
  // consecutive padded rows at the same offset
  const int tok = tid & 63, part = tid >> 6;
  constexpr int HD = D / NPART;
  // PV mapping: thread -> (token group = tid / 16 (TPG tokens), dim group = tid % 16 (D/16 dims))
  constexpr int DG = D / 16;
  const int tg = tid >> 4, dg = tid & 15;
  float acc[G][DG];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int i = 0; i < DG; ++i) acc[g][i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;  // maintained by warp g (lane-uniform) for head g
  if (G > NT / 32 && tid < G) {
    s_m[tid] = -INFINITY;
    s_l[tid] = 0.f;
  }

  // prologue: two tiles in flight. Every iteration commits exactly one group (possibly empty),
  // so "all but the two newest groups are complete" always means "this iteration's tile landed".
  if (start < end) load_tile(0, start); else cp_async_commit_group();
  if (start + TILE < end) load_tile(1, start + TILE); else cp_async_commit_group();
  int stage = 0;
  for (int t0 = start; t0 < end; t0 += TILE, stage = (stage + 1 == S::kStages) ? 0 : stage + 1) {
    if (t0 + 2 * TILE < end) {
      load_tile((stage + 2) % S::kStages, t0 + 2 * TILE);
    } else {
      cp_async_commit_group();
    }
    cp_async_wait_group_n<2>();
    __syncthreads();
    const __nv_bfloat16* sk = ring + stage * S::kStageElems;
    const __nv_bfloat16* sv = sk + TILE * ROW;
    // ---- scores: NPART threads per token, each over a slice of the head dim
    {
      const int t = t0 + tok;
      float dot[G];
#pragma unroll
      for (int g = 0; g < G; ++g) dot[g] = 0.f;
      const uint4* kp = reinterpret_cast<const uint4*>(sk + tok * ROW + part * HD);
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
        const uint4 raw = kp[c];
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float kf[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 kv = __bfloat1622float2(h2[j]);
          kf[2 * j] = kv.x;
          kf[2 * j + 1] = kv.y;
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float4 qa = *reinterpret_cast<const float4*>(&s_q[g][part * HD + c * 8]);
          const float4 qb = *reinterpret_cast<const float4*>(&s_q[g][part * HD + c * 8 + 4]);
          dot[g] += qa.x * kf[0] + qa.y * kf[1] + qa.z * kf[2] + qa.w * kf[3] + qb.x * kf[4] +
                    qb.y * kf[5] + qb.z * kf[6] + qb.w * kf[7];
        }
      }
      // the slices of a token sit 64 threads apart: combine through shared memory
#pragma unroll
      for (int g = 0; g < G; ++g) s_part[part][g][tok] = dot[g];
      __syncthreads();
      if (part == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float sum = 0.f;
#pragma unroll
          for (int pp = 0; pp < NPART; ++pp) sum += s_part[pp][g][tok];
          s_scores[g][tok] = (t < end) ? sum : -INFINITY;
        }
      }
    }
    __syncthreads();
    // ---- online softmax statistics: warp g owns head g (G <= 4 warps; loop otherwise)
    for (int g = warp; g < G; g += NT / 32) {
      const float a0 = s_scores[g][lane], a1 = s_scores[g][lane + 32];
      const float tmax = warp_max_f(fmaxf(a0, a1));
      // m_run / l_run live in registers of warp (g % 4); with G > 4 they are kept in smem below
      float m_old = (G <= NT / 32) ? m_run : s_m[g];
      float l_old = (G <= NT / 32) ? l_run : s_l[g];
      const float m_new = fmaxf(m_old, tmax);
      const float alpha = (m_old == -INFINITY) ? 0.f : exp2f(m_old - m_new);
      const float p0 = (a0 == -INFINITY) ? 0.f : exp2f(a0 - m_new);
      const float p1 = (a1 == -INFINITY) ? 0.f : exp2f(a1 - m_new);
      s_scores[g][lane] = p0;
      s_scores[g][lane + 32] = p1;
      const float l_new = l_old * alpha + warp_sum_f(p0 + p1);
      if (G <= NT / 32) { m_run = m_new; l_run = l_new; } else if (lane == 0) { s_m[g] = m_new; s_l[g] = l_new; }
      if (lane == 0) s_alpha[g] = alpha;
    }
    __syncthreads();
    // ---- P V
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float al = s_alpha[g];
#pragma unroll
      for (int i = 0; i < DG; ++i) acc[g][i] *= al;
    }
#pragma unroll
    for (int j = 0; j < TPG; ++j) {
      const int tl = tg * TPG + j;
      if (t0 + tl < end) {
        const __nv_bfloat16* vp = sv + tl * ROW + dg * DG;
        float vv[DG];
        if (DG == 8) {
          const uint4 raw = *reinterpret_cast<const uint4*>(vp);
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h2[i]);
            vv[2 * i] = f.x;
            vv[2 * i + 1] = f.y;
          }
        } else {
          const uint2 raw = *reinterpret_cast<const uint2*>(vp);
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int i = 0; i < DG / 2; ++i) {
            const float2 f = __bfloat1622float2(h2[i]);
            vv[2 * i] = f.x;
            vv[2 * i + 1] = f.y;
          }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float p = s_scores[g][tl];
#pragma unroll
          for (int i = 0; i < DG; ++i) acc[g][i] += p * vv[i];
        }
      }
    }
    __syncthreads();   // everyone is done with this stage before the next iteration refills it
  }

  // ---- reduce the 8 token groups, write the split's partial result
  cp_async_wait_group_n<0>();
  __syncthreads();
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int i = 0; i < DG; ++i) s_red[tg][g][dg * DG + i] = acc[g][i];
  if (G <= NT / 32 && warp < G && lane == 0) {
    s_scores[warp][0] = m_run;
    s_scores[warp][1] = l_run;
  }
  __syncthreads();
  for (int idx = tid; idx < G * D; idx += NT) {
    const int g = idx / D, d = idx - g * D;
    float o = 0.f;
#pragma unroll
    for (int j = 0; j < NTG; ++j) o += s_red[j][g][d];
    const float m = (G <= NT / 32) ? s_scores[g][0] : s_m[g];
    const float l = (G <= NT / 32) ? s_scores[g][1] : s_l[g];
    const int h = kh * G + g;
    if (splits == 1) {
      out[(static_cast<long>(b) * hq + h) * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    } else {
      float* w = ws + ((static_cast<long>(b) * hq + h) * splits + sp) * (D + 2);
      w[d] = o;
      if (d == 0) {
        w[D] = m;
        w[D + 1] = l;
      }
    }
  }
}

// out[b, h, :] = sum_s exp2(m_s - M) o_s / sum_s exp2(m_s - M) l_s
template <int D>
__global__ void decode_merge_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ out,
                                    int splits) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // a dependent launch may set itself up under this kernel
  const long bh = blockIdx.x;
  const float* w = ws + bh * splits * (D + 2);
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, w[s * (D + 2) + D]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.f, l = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float m = w[s * (D + 2) + D];
      const float f = (m == -INFINITY) ? 0.f : exp2f(m - M);
      o += f * w[s * (D + 2) + d];
      l += f * w[s * (D + 2) + D + 1];
    }
    out[bh * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
  }
}

// ------------------------------------------------------------------ prefill attention
// Tensor-core tiles (mma.sync m16n8k16, bf16 in / fp32 accumulate): 64 query rows per CTA
// (4 warps x 16 rows), 64 keys per step, online softmax in registers. grid (batch * q_tiles,
// query heads). Keys are gathered from pages with cp.async. Shared-memory rows are 16-byte-
// chunk XOR-swizzled by (row % 8).
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int n = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;"); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                          uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int D>
__global__ void __launch_bounds__(128)
paged_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                     const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out,
                     const int* __restrict__ page_table, const int* __restrict__ req_slots,
                     const int* __restrict__ qo_indptr, const int* __restrict__ seq_lens, int hq,
                     int hk, int max_pages, int q_tiles, long q_stride, long o_stride,
                     float scale_log2, long num_pages, int* __restrict__ status) {
  constexpr int BM = 64, BN = 64, CH = D / 8;  // CH: 16-byte chunks per row
  extern __shared__ __align__(16) uint8_t smem[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem);
  __nv_bfloat16* sK = sQ + BM * D;
  __nv_bfloat16* sV = sK + BN * D;

  const int b = blockIdx.x / q_tiles, mt = blockIdx.x % q_tiles;
  const int h = blockIdx.y, kh = h / (hq / hk);
  const int q0 = qo_indptr[b], ext = qo_indptr[b + 1] - q0;
  const int m0 = mt * BM;
  if (m0 >= ext) return;
  const int seq = seq_lens[b];
  const int prefix = seq - ext;
  const int* pt = page_table + static_cast<long>(req_slots[b]) * max_pages;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t sQa = static_cast<uint32_t>(__cvta_generic_to_shared(sQ));
  const uint32_t sKa = static_cast<uint32_t>(__cvta_generic_to_shared(sK));
  const uint32_t sVa = static_cast<uint32_t>(__cvta_generic_to_shared(sV));

  // ---- Q tile -> smem (rows beyond the request read as zeros)
  for (int i = tid; i < BM * CH; i += 128) {
    const int r = i / CH, c = i % CH;
    const bool ok = m0 + r < ext;
    const __nv_bfloat16* src = q + static_cast<long>(q0 + m0 + (ok ? r : 0)) * q_stride + h * D + c * 8;
    cp_async16(sQa + (r * CH + (c ^ (r & 7))) * 16, src, ok);
  }
  cp_async_commit();

  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int row_in_warp = lane >> 2;              // rows r and r + 8 of the warp's 16
  const int qpos0 = prefix + m0 + warp * 16 + row_in_warp;
  const int kv_end = min(seq, prefix + m0 + BM);  // causal: nothing beyond the tile's last query

  uint32_t qf[D / 16][4];
  bool q_loaded = false;

  for (int n0 = 0; n0 < kv_end; n0 += BN) {
    __syncthreads();  // previous tile's reads of sK / sV are done
    for (int i = tid; i < BN * CH; i += 128) {
      const int r = i / CH, c = i % CH;
      const int t = n0 + r;
      const bool ok = t < seq;
      int pg = ok ? ((t >> 4) < max_pages ? pt[t >> 4] : -1) : 0;
      if (pg < 0 || pg >= num_pages) {
        if (status) atomicCAS(status, 0, kBadPageId);      // reported, and read from the scratch page
        pg = 0;
      }
      const long slot = static_cast<long>(pg) * kPage + (t & 15);
      const long off = (slot * hk + kh) * D + c * 8;
      cp_async16(sKa + (r * CH + (c ^ (r & 7))) * 16, k_cache + off, ok);
      cp_async16(sVa + (r * CH + (c ^ (r & 7))) * 16, v_cache + off, ok);
    }
    cp_async_commit();
    cp_async_wait_all();
    __syncthreads();
    if (!q_loaded) {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = ks * 2 + (lane >> 4);
        ldsm_x4(sQa + (r * CH + (c ^ (r & 7))) * 16, qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
      }
      q_loaded = true;
    }
    // ---- S = Q K^T  (16 x 64 per warp)
    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int nb = 0; nb < BN / 8; nb += 2) {
        // matrices: (keys nb*8.., dims ks*16..+7), (same keys, dims +8), (keys +8, dims lo), (keys +8, dims hi)
        const int r = nb * 8 + (lane & 7) + ((lane >> 4) & 1) * 8;
        const int c = ks * 2 + ((lane >> 3) & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(sKa + (r * CH + (c ^ (r & 7))) * 16, b0, b1, b2, b3);
        mma_bf16(s[nb], qf[ks], b0, b1);
        mma_bf16(s[nb + 1], qf[ks], b2, b3);
      }
    }
    // ---- mask + online softmax (thread holds rows r, r + 8; cols nb*8 + (lane%4)*2 + {0,1})
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = n0 + nb * 8 + (lane & 3) * 2 + (j & 1);
        const int qp = qpos0 + (j >> 1) * 8;
        const bool ok = col <= qp && col < seq;
        s[nb][j] = ok ? s[nb][j] * scale_log2 : -INFINITY;
        tmax[j >> 1] = fmaxf(tmax[j >> 1], s[nb][j]);
      }
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
      tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
      const float m_new = fmaxf(m_run[r], tmax[r]);
      alpha[r] = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - m_new);
      m_run[r] = m_new;
    }
    float rsum[2] = {0.f, 0.f};
    uint32_t pf[BN / 16][4];
#pragma unroll
    for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float mref = m_run[j >> 1];
        const float p = (s[nb][j] == -INFINITY || mref == -INFINITY) ? 0.f : exp2f(s[nb][j] - mref);
        s[nb][j] = p;
        rsum[j >> 1] += p;
      }
      // accumulator layout of two adjacent 8-wide blocks == A fragment of one 16-wide k block
      if (nb & 1) {
        const int kb = nb >> 1;
        pf[kb][0] = pack2(s[nb - 1][0], s[nb - 1][1]);
        pf[kb][1] = pack2(s[nb - 1][2], s[nb - 1][3]);
        pf[kb][2] = pack2(s[nb][0], s[nb][1]);
        pf[kb][3] = pack2(s[nb][2], s[nb][3]);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rsum[r] += __shfl_xor_sync(0xffffffffu, rsum[r], 1);
      rsum[r] += __shfl_xor_sync(0xffffffffu, rsum[r], 2);
      l_run[r] = l_run[r] * alpha[r] + rsum[r];
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o_acc[i][0] *= alpha[0];
      o_acc[i][1] *= alpha[0];
      o_acc[i][2] *= alpha[1];
      o_acc[i][3] *= alpha[1];
    }
    // ---- O += P V
#pragma unroll
    for (int kb = 0; kb < BN / 16; ++kb) {
#pragma unroll
      for (int db = 0; db < D / 8; db += 2) {
        // transposed loads: (tokens kb*16.., dims db*8..), (tokens +8, same dims), then dims +8
        const int r = kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = db + (lane >> 4);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(sVa + (r * CH + (c ^ (r & 7))) * 16, b0, b1, b2, b3);
        mma_bf16(o_acc[db], pf[kb], b0, b1);
        mma_bf16(o_acc[db + 1], pf[kb], b2, b3);
      }
    }
  }

  // ---- normalise and store
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = m0 + warp * 16 + row_in_warp + r * 8;
    if (row < ext) {
      const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
      __nv_bfloat16* op = out + static_cast<long>(q0 + row) * o_stride + h * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        const int col = i * 8 + (lane & 3) * 2;
        *reinterpret_cast<uint32_t*>(op + col) = pack2(o_acc[i][r * 2] * inv, o_acc[i][r * 2 + 1] * inv);
      }
    }
  }
}

// ------------------------------------------------------------------ sampling
// One CTA per row: argmax_i (x_i / T + Gumbel_i) is a draw from softmax(x / T); the same pass
// keeps the running log-sum-exp so the log-probability of the draw needs no second pass.
__device__ __forceinline__ uint32_t mix32(uint64_t x) {
  x ^= x >> 33;
  x *= 0xff51afd7ed558ccdULL;
  x ^= x >> 33;
  x *= 0xc4ceb9fe1a85ec53ULL;
  x ^= x >> 33;
  return static_cast<uint32_t>(x);
}

__global__ void __launch_bounds__(1024)
sample_gumbel_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                     const bool* __restrict__ greedy, int64_t* __restrict__ ids,
                     float* __restrict__ logprobs, int vocab, long ld, uint64_t seed,
                     uint64_t call) {
  __shared__ float r_val[32], r_m[32], r_s[32], r_x[32];
  __shared__ int r_idx[32];
  const long row = blockIdx.x;
  const float* x = logits + row * ld;
  const float inv_t = 1.f / fmaxf(temperature[row], 1e-6f);
  const bool g = greedy[row];
  const uint64_t base = (seed * 0x9E3779B97F4A7C15ULL) ^ (call * 0xD1B54A32D192ED03ULL) ^
                        (static_cast<uint64_t>(row) << 32);
  float best = -INFINITY, best_x = 0.f, m = -INFINITY, s = 0.f;
  int best_i = 0;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    float v = x[i];
    if (v != v) v = -1e5f;  // NaN guard
    v *= inv_t;
    float noisy = v;
    if (!g) {
      const uint32_t u32 = mix32(base + static_cast<uint64_t>(i));
      const float u = (static_cast<float>(u32 >> 8) + 0.5f) * (1.f / 16777216.f);
      noisy = v - __logf(-__logf(u));
    }
    if (noisy > best) { best = noisy; best_i = i; best_x = v; }
    if (v > m) { s = s * __expf(m - v) + 1.f; m = v; } else { s += __expf(v - m); }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    const float ox = __shfl_xor_sync(0xffffffffu, best_x, o);
    if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; best_x = ox; }
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float os = __shfl_xor_sync(0xffffffffu, s, o);
    const float mm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - mm)) + (om == -INFINITY ? 0.f : os * __expf(om - mm));
    m = mm;
  }
  if (lane == 0) { r_val[warp] = best; r_idx[warp] = best_i; r_x[warp] = best_x; r_m[warp] = m; r_s[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? r_val[lane] : -INFINITY;
    best_i = lane < nw ? r_idx[lane] : 0;
    best_x = lane < nw ? r_x[lane] : 0.f;
    m = lane < nw ? r_m[lane] : -INFINITY;
    s = lane < nw ? r_s[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      const float ox = __shfl_xor_sync(0xffffffffu, best_x, o);
      if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; best_x = ox; }
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const float os = __shfl_xor_sync(0xffffffffu, s, o);
      const float mm = fmaxf(m, om);
      s = (m == -INFINITY ? 0.f : s * __expf(m - mm)) + (om == -INFINITY ? 0.f : os * __expf(om - mm));
      m = mm;
    }
    if (lane == 0) {
      ids[row] = best_i;
      logprobs[row] = best_x - (m + __logf(s));
    }
  }
}

}  // namespace

// ------------------------------------------------------------------ launchers
cudaError_t rope_append(const RopeAppendArgs& a, cudaStream_t stream) {
  if (a.tokens == 0) return cudaSuccess;
  if (a.dim % 8 || a.rot % 2 || a.rot > a.dim || (a.dim - a.rot) % 2 || a.v_stride % 8)
    return cudaErrorInvalidValue;
  rope_append_kernel<<<a.tokens, 256, 0, stream>>>(
      static_cast<__nv_bfloat16*>(a.q), static_cast<const __nv_bfloat16*>(a.k),
      static_cast<const __nv_bfloat16*>(a.v), static_cast<__nv_bfloat16*>(a.k_cache),
      static_cast<__nv_bfloat16*>(a.v_cache), a.cos, a.sin, a.positions, a.out_loc, a.hq, a.hk,
      a.dim, a.rot, a.q_stride, a.k_stride, a.v_stride, a.interleaved ? 1 : 0, a.cache_slots);
  return cudaGetLastError();
}

int paged_decode_splits(int batch, int hk, int sm_count) {
  int s = (4 * sm_count + batch * hk - 1) / (batch * hk);
  if (s < 1) s = 1;
  if (s > 32) s = 32;
  return s;
}

template <int D, int G>
static cudaError_t launch_decode(const PagedDecodeArgs& a, cudaStream_t stream) {
  dim3 grid(a.batch, a.hk, a.splits);
  constexpr int smem = DecodeSmem<D>::kBytes;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(paged_decode_kernel<D, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  paged_decode_kernel<D, G><<<grid, kDecodeThreads, smem, stream>>>(
      static_cast<const __nv_bfloat16*>(a.q), static_cast<const __nv_bfloat16*>(a.k_cache),
      static_cast<const __nv_bfloat16*>(a.v_cache), a.page_table, a.req_slots, a.seq_lens, a.workspace,
      static_cast<__nv_bfloat16*>(a.out), a.hq, a.hk, a.max_pages, a.splits, a.q_stride,
      a.scale * 1.4426950408889634f, a.num_pages, a.status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || a.splits == 1) return e;
  decode_merge_kernel<D><<<a.batch * a.hq, D, 0, stream>>>(a.workspace, static_cast<__nv_bfloat16*>(a.out), a.splits);
  return cudaGetLastError();
}

cudaError_t paged_decode(const PagedDecodeArgs& a, cudaStream_t stream) {
  if (a.batch == 0) return cudaSuccess;
  if (a.hq % a.hk) return cudaErrorInvalidValue;
  const int g = a.hq / a.hk;
  if (a.splits > 1 && !a.workspace) return cudaErrorInvalidValue;
#define HB_DECODE(DD, GG) if (a.dim == DD && g == GG) return launch_decode<DD, GG>(a, stream);
  HB_DECODE(128, 1) HB_DECODE(128, 2) HB_DECODE(128, 3) HB_DECODE(128, 4) HB_DECODE(128, 8)
  HB_DECODE(64, 1) HB_DECODE(64, 2) HB_DECODE(64, 4) HB_DECODE(64, 8)
#undef HB_DECODE
  return cudaErrorInvalidValue;
}

cudaError_t paged_prefill(const PagedPrefillArgs& a, cudaStream_t stream) {
  if (a.batch == 0 || a.max_extend == 0) return cudaSuccess;
  if (a.hq % a.hk || (a.dim != 64 && a.dim != 128) || a.q_stride % 8 || a.o_stride % 2)
    return cudaErrorInvalidValue;
  const int q_tiles = (a.max_extend + 63) / 64;
  dim3 grid(a.batch * q_tiles, a.hq);
  const int smem = 3 * 64 * a.dim * 2;
  const float sl2 = a.scale * 1.4426950408889634f;
  auto Q = static_cast<const __nv_bfloat16*>(a.q);
  auto K = static_cast<const __nv_bfloat16*>(a.k_cache);
  auto V = static_cast<const __nv_bfloat16*>(a.v_cache);
  auto O = static_cast<__nv_bfloat16*>(a.out);
  if (a.dim == 128) {
    static bool set = false;
    if (!set) {
      cudaError_t e = cudaFuncSetAttribute(paged_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return e;
      set = true;
    }
    paged_prefill_kernel<128><<<grid, 128, smem, stream>>>(Q, K, V, O, a.page_table, a.req_slots, a.qo_indptr,
                                                           a.seq_lens, a.hq, a.hk, a.max_pages, q_tiles,
                                                           a.q_stride, a.o_stride, sl2, a.num_pages, a.status);
  } else {
    paged_prefill_kernel<64><<<grid, 128, smem, stream>>>(Q, K, V, O, a.page_table, a.req_slots, a.qo_indptr,
                                                          a.seq_lens, a.hq, a.hk, a.max_pages, q_tiles,
                                                          a.q_stride, a.o_stride, sl2, a.num_pages, a.status);
  }
  return cudaGetLastError();
}

cudaError_t sample_gumbel(const float* logits, const float* temperature, const bool* greedy,
                          int64_t* ids, float* logprobs, int rows, int vocab, long ld, uint64_t seed,
                          uint64_t call, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  sample_gumbel_kernel<<<rows, 1024, 0, stream>>>(logits, temperature, greedy, ids, logprobs, vocab, ld,
                                                  seed, call);
  return cudaGetLastError();
}

}  // namespace hb
