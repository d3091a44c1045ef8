// Training attention for sm_100a: softmax(mask(scale * Q K^T)) V and its gradients on tcgen05
// tensor cores with the score / probability tiles held in tensor memory.
//
// Forward (`attn_fwd_kernel`): one CTA per 256 query rows of one head, 320 threads:
//   warp 0 (one lane)   TMA producer: the two 128-row Q tiles once, then K_j, V_j tiles through
//                       a shared-memory ring (cp.async.bulk.tensor, 128B swizzle, no multicast)
//   warp 1 (one lane)   MMA issuer: S_t = Q_t K_j^T into TMEM, O_t += P_t V_j with P_t read from
//                       TMEM (it overwrites the first half of S_t's columns as bf16)
//   warp 0 (all lanes)  TMEM allocation (all 512 columns: S_0 S_1 O_0 O_1)
//   warps 2-5 / 6-9     softmax of tile 0 / tile 1: one thread per query row, online softmax
//                       with deferred rescaling (O_t is only rescaled when a row's maximum grew
//                       by more than 2^8), P_t written back to TMEM with tcgen05.st in two halves
//                       so that O_t += P_t V_j starts on the first half
// While one tile's rows are in the softmax, the tensor cores work on the other tile.
//
// Backward (`attn_bwd_kernel`): one CTA per 128 key/value rows of one KV head; it walks the query
// tiles (of every query head of the group) that can see those rows and keeps dK, dV in TMEM:
//   S^T = K Q^T, dP^T = V dO^T         (TMEM; one thread per key row reads them)
//   P^T = exp2(S^T c - lse)            -> TMEM (bf16, inside S^T's columns), A operand of dV += P^T dO
//   dS^T = P^T (dP^T - delta) scale    -> shared memory, read K-major by dK += dS^T Q and
//                                         MN-major by dQ = dS K
//   dQ tile                            -> TMEM (over dP^T) -> shared memory -> bulk tensor reductions
//                                         (fp32 add, whole 128-byte lines) into dq_accum
//
// Masks (causal, sliding window, segment bounds for packed sequences / documents, soft-capping)
// are evaluated from per-token bounds on the device; nothing depends on host-side lengths.
//
// Replaces the FlashAttention-2 / SDPA / FlexAttention calls of the reference
// (transformers/attention.py:505-558, 600-643).
#include "attention.h"

#include <math.h>
#include <stdio.h>

#include <algorithm>

#include "sm100.cuh"

namespace hb {

namespace {

constexpr int kTile = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.f;   // in log2 units: P values stay below 2^8

struct AttnParams {
  int total;
  int n_heads, n_kv_heads;
  int seq_len;
  const int* seg_start;
  const int* seg_end;
  int causal;
  int window;
  float scale;
  float softcap;
  int* status;
};

// ---------------------------------------------------------------- extra tcgen05 forms
// Shared-memory matrix descriptors, split in halves: every operand tile here uses the 128-byte
// swizzle with 1024 bytes between 8-row groups, so the high word is one constant and the low word
// is (address >> 4) | (bytes between 64-wide chunks >> 4) << 16. Stepping an operand along K adds
// a constant to the low word, which keeps the issuing thread's instruction stream short.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr & 0x3ffffu) >> 4) | (((lbo_bytes >> 4) & 0x3fffu) << 16);
}
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(tmem_d),
      "r"(a_lo), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
      "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
      "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Segment of token t: [s0, s1).
__device__ __forceinline__ void segment_of(const AttnParams& p, int t, int& s0, int& s1) {
  if (p.seg_start) {
    s0 = p.seg_start[t];
    s1 = p.seg_end[t];
  } else {
    s0 = (t / p.seq_len) * p.seq_len;
    s1 = min(s0 + p.seq_len, p.total);
  }
}
// Keys that query row q may attend: [lo, hi] (empty when hi < lo).
__device__ __forceinline__ void query_bounds(const AttnParams& p, int q, int& lo, int& hi) {
  if (q >= p.total) {
    lo = 0;
    hi = -1;
    return;
  }
  int s0, s1;
  segment_of(p, q, s0, s1);
  lo = s0;
  hi = p.causal ? q : s1 - 1;
  if (p.window > 0) lo = max(lo, q - p.window + 1);     // the window limits how far back a query looks
}
// Queries that may attend key row k: [lo, hi].
__device__ __forceinline__ void key_bounds(const AttnParams& p, int k, int& lo, int& hi) {
  if (k >= p.total) {
    lo = 0;
    hi = -1;
    return;
  }
  int s0, s1;
  segment_of(p, k, s0, s1);
  lo = p.causal ? k : s0;
  hi = s1 - 1;
  if (p.window > 0) hi = min(hi, k + p.window - 1);
}

// ================================================================== forward
template <int D>
struct FwdCfg {
  static constexpr int kChunks = D / 64;                 // 64-element (128-byte) column chunks
  static constexpr int kChunkBytes = kTile * 128;        // 128 rows x 128 bytes
  static constexpr int kTileBytes = kChunks * kChunkBytes;
  static constexpr int kStages = (D == 128) ? 4 : 6;
  static constexpr int kSmemBytes = (2 + kStages) * kTileBytes + 1024;
  static constexpr int kThreads = 320;
  static constexpr int kTmemCols = 512;
  static constexpr int kOCol = 256;                       // O_t at kOCol + t * D
};

template <int D, bool kSoftcap>
__global__ void __launch_bounds__(320, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, __nv_bfloat16* __restrict__ out,
                float* __restrict__ lse, const __grid_constant__ AttnParams p) {
  using C = FwdCfg<D>;
  constexpr int kStages = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_q_full[2];
  __shared__ __align__(8) uint64_t bar_kv_full[kStages];
  __shared__ __align__(8) uint64_t bar_kv_empty[kStages];
  __shared__ __align__(8) uint64_t bar_s_full[2];
  __shared__ __align__(8) uint64_t bar_p_ready[2][2];   // [tile][half]: one phase per key tile each, so the
                                                        // softmax never runs two phases ahead of the waiter
  __shared__ __align__(8) uint64_t bar_o_full[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  // a launch whose status word already reports a failed wait does nothing: a protocol error then
  // costs one wait budget, not one per CTA
  if (threadIdx.x == 0) abort_flag = p.status ? *reinterpret_cast<volatile int*>(p.status) : 0;
  __syncthreads();
  if (abort_flag) return;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem[2] = {smem_base, smem_base + C::kTileBytes};
  const uint32_t ring = smem_base + 2 * C::kTileBytes;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- which 256 query rows, which head (heaviest blocks first)
  const int H = p.n_heads;
  int qb, head;
  {
    const int id = blockIdx.x;
    if (!p.seg_start && p.seq_len % 256 == 0 && p.total % p.seq_len == 0) {
      const int per_seq = p.seq_len / 256, nseq = p.total / p.seq_len;
      const int pos = per_seq - 1 - id / (nseq * H);
      const int rem = id % (nseq * H);
      qb = (rem / H) * per_seq + pos;
      head = rem % H;
    } else {
      const int nqb = (p.total + 255) / 256;
      qb = nqb - 1 - id / H;
      head = id % H;
    }
  }
  const int kv_head = head / (H / p.n_kv_heads);
  // ---- key tile range of each query tile
  int jb[2], je[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r0 = qb * 256 + t * kTile;
    if (r0 >= p.total) {
      jb[t] = je[t] = 0;
      continue;
    }
    int lo, hi, lo2, hi2;
    query_bounds(p, r0, lo, hi2);
    query_bounds(p, min(r0 + kTile - 1, p.total - 1), lo2, hi);
    jb[t] = lo / kTile;
    je[t] = hi / kTile + 1;
  }
  const bool act1 = je[1] > jb[1];
  const int J0 = act1 ? min(jb[0], jb[1]) : jb[0];
  const int J1 = act1 ? max(je[0], je[1]) : je[0];

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int t = 0; t < 2; ++t) {
      mbar_init(smem_u32(&bar_q_full[t]), 1);
      mbar_init(smem_u32(&bar_s_full[t]), 1);
      mbar_init(smem_u32(&bar_p_ready[t][0]), 4);
      mbar_init(smem_u32(&bar_p_ready[t][1]), 4);
      mbar_init(smem_u32(&bar_o_full[t]), 1);
    }
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_kv_full[s]), 1);
      mbar_init(smem_u32(&bar_kv_empty[s]), 1);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ producer
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      if (je[t] <= jb[t]) continue;
      const uint32_t full = smem_u32(&bar_q_full[t]);
      mbar_expect_tx(full, C::kTileBytes);
#pragma unroll
      for (int c = 0; c < C::kChunks; ++c)
        tma_load_3d(q_smem[t] + c * C::kChunkBytes, &tm_q, full, c * 64, head, qb * 256 + t * kTile);
    }
    int e = 0;
    bool ok = true;
    for (int j = J0; j < J1 && ok; ++j) {
#pragma unroll
      for (int which = 0; which < 2; ++which, ++e) {
        const int stage = e % kStages;
        const uint32_t phase = (e / kStages) & 1;
        ok = mbar_wait(smem_u32(&bar_kv_empty[stage]), phase ^ 1, &abort_flag, p.status, kTimeoutEmpty);
        if (!ok) break;
        const uint32_t full = smem_u32(&bar_kv_full[stage]);
        mbar_expect_tx(full, C::kTileBytes);
        const uint32_t dst = ring + stage * C::kTileBytes;
#pragma unroll
        for (int c = 0; c < C::kChunks; ++c)
          tma_load_3d(dst + c * C::kChunkBytes, which == 0 ? &tm_k : &tm_v, full, c * 64, kv_head, j * kTile);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_qk = make_idesc_bf16(kTile, kTile, false, false);
    constexpr uint32_t idesc_pv = make_idesc_bf16(kTile, D, false, true);
    bool ok = true;
    const uint32_t q_lo[2] = {desc_lo(q_smem[0], 0), desc_lo(q_smem[1], 0)};
    auto issue_s = [&](int t, uint32_t k_addr) {
      const uint32_t k_lo = desc_lo(k_addr, 0);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t off = static_cast<uint32_t>(((ks >> 2) * C::kChunkBytes + (ks & 3) * 32) >> 4);
        umma_ss(tmem_base + t * kTile, q_lo[t] + off, k_lo + off, idesc_qk, ks != 0);
      }
      umma_commit(smem_u32(&bar_s_full[t]));
    };
    // O_t += P_t V_j for one half of the key tile (P arrives in two halves of 64 keys, so the
    // first product runs while the second half is still in the exponentials)
    auto issue_pv = [&](int t, uint32_t v_addr, bool acc, int half) {
      const uint32_t v_lo = desc_lo(v_addr, C::kChunkBytes);
#pragma unroll
      for (int k4 = 0; k4 < kTile / 32; ++k4) {
        const int ks = half * (kTile / 32) + k4;
        umma_ts(tmem_base + C::kOCol + t * D, tmem_base + t * kTile + ks * 8,
                v_lo + static_cast<uint32_t>((ks * 2048) >> 4), idesc_pv, acc || ks != 0);
      }
    };
    auto wait_entry = [&](int e) -> bool {
      return mbar_wait(smem_u32(&bar_kv_full[e % kStages]), (e / kStages) & 1, &abort_flag, p.status,
                       kTimeoutFull);
    };
    auto entry_addr = [&](int e) -> uint32_t { return ring + (e % kStages) * C::kTileBytes; };
    for (int t = 0; t < 2 && ok; ++t)
      if (je[t] > jb[t]) ok = mbar_wait(smem_u32(&bar_q_full[t]), 0, &abort_flag, p.status, kTimeoutFull);
    uint32_t n_p[2] = {0, 0};
    if (ok && J1 > J0) {
      ok = wait_entry(0);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < 2; ++t)
          if (jb[t] <= J0 && J0 < je[t]) issue_s(t, entry_addr(0));
        umma_commit(smem_u32(&bar_kv_empty[0]));
      }
    }
    for (int j = J0; j < J1 && ok; ++j) {
      const int e_v = 2 * (j - J0) + 1, e_kn = e_v + 1;
      const bool next = j + 1 < J1;
      ok = wait_entry(e_v);
      if (!ok) break;
      bool have_next = false;
      for (int t = 0; t < 2 && ok; ++t) {
        if (jb[t] <= j && j < je[t]) {
          for (int half = 0; half < 2 && ok; ++half) {
            ok = mbar_wait(smem_u32(&bar_p_ready[t][half]), n_p[t] & 1, &abort_flag, p.status, kTimeoutTmemEmpty);
            if (!ok) break;
            tc_fence_after();
            issue_pv(t, entry_addr(e_v), j > jb[t], half);
          }
          if (!ok) break;
          ++n_p[t];
          if (j == je[t] - 1) umma_commit(smem_u32(&bar_o_full[t]));
        }
        if (next && jb[t] <= j + 1 && j + 1 < je[t]) {
          if (!have_next) {
            ok = wait_entry(e_kn);
            if (!ok) break;
            have_next = true;
            tc_fence_after();
          }
          issue_s(t, entry_addr(e_kn));
        }
      }
      if (!ok) break;
      umma_commit(smem_u32(&bar_kv_empty[e_v % kStages]));
      if (next) {
        if (!have_next) ok = wait_entry(e_kn);
        if (ok) umma_commit(smem_u32(&bar_kv_empty[e_kn % kStages]));
      }
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------ softmax + epilogue
    // warps 2-5 own query tile 0, warps 6-9 tile 1; a warp reads the TMEM lane quarter warp % 4
    const int t = (warp - 2) >> 2;
    const int wq = warp & 3;
    if (je[t] > jb[t]) {
      const int row = qb * 256 + t * kTile + wq * 32 + lane;
      int lo, hi;
      query_bounds(p, row, lo, hi);
      const uint32_t lane_addr = static_cast<uint32_t>(wq * 32) << 16;
      const uint32_t s_addr = tmem_base + t * kTile + lane_addr;
      const uint32_t o_addr = tmem_base + C::kOCol + t * D + lane_addr;
      const float c2 = kSoftcap ? kLog2e : p.scale * kLog2e;   // multiplies a (capped) score into log2 units
      const float cap_in = kSoftcap ? p.scale / p.softcap : 0.f;
      float m_used = -INFINITY, l = 0.f;
      bool ok = true;
      int k = 0;
      for (int j = jb[t]; j < je[t]; ++j, ++k) {
        ok = mbar_wait(smem_u32(&bar_s_full[t]), k & 1, &abort_flag, p.status, kTimeoutTmemFull);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const int kv0 = j * kTile;
        const bool mask_tile = __any_sync(0xffffffffu, kv0 < lo || kv0 + kTile - 1 > hi);
        // ---- the whole score row into registers
        uint32_t v[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_32x32(s_addr + c * 32, v[c]);
        tmem_ld_wait();
        if (kSoftcap) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              v[c][i] = __float_as_uint(p.softcap * tanh_fast(__uint_as_float(v[c][i]) * cap_in));
        }
        if (mask_tile) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int kv = kv0 + c * 32 + i;
              if (kv < lo || kv > hi) v[c][i] = __float_as_uint(-INFINITY);
            }
        }
        // ---- row maximum (eight independent chains)
        float mx[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) mx[u] = -INFINITY;
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) mx[i & 7] = fmaxf(mx[i & 7], __uint_as_float(v[c][i]));
        const float mt = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])),
                               fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
        // ---- deferred rescaling of the running output
        const float m_new = fmaxf(m_used, mt);
        float m_next = m_used;
        if (k == 0 || (m_new - m_used) * c2 > kRescaleThreshold) m_next = m_new;
        const bool rescale = k != 0 && m_next != m_used;
        if (__any_sync(0xffffffffu, rescale)) {
          const float alpha = (m_next == m_used) ? 1.f : exp2f((m_used - m_next) * c2);
          l *= alpha;
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(o_addr + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(o_addr + c * 32, o);
          }
          tmem_st_wait();
        }
        m_used = m_next;
        const float mc = (m_used == -INFINITY) ? 0.f : m_used * c2;
        // ---- P = exp2(S c2 - m c2) as bf16 pairs over the first half of S's columns
        float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float e0 = ex2_fast(fmaf(__uint_as_float(v[c][2 * i]), c2, -mc));
            const float e1 = ex2_fast(fmaf(__uint_as_float(v[c][2 * i + 1]), c2, -mc));
            ls[i & 3] += e0 + e1;
            pk[i] = pack_bf16x2(e0, e1);
          }
          tmem_st_32x16(s_addr + c * 16, pk);
          if (c & 1) {
            // one half of P (64 keys) is complete: hand it to the tensor cores
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_p_ready[t][c >> 1]));
          }
        }
        l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      }
      if (ok) {
        ok = mbar_wait(smem_u32(&bar_o_full[t]), 0, &abort_flag, p.status, kTimeoutTmemFull);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const bool live = row < p.total;
        __nv_bfloat16* dst = out + (static_cast<size_t>(row) * H + head) * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(o_addr + c * 32, v);
          tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(v[8 * g]) * inv, __uint_as_float(v[8 * g + 1]) * inv);
              o.y = pack_bf16x2(__uint_as_float(v[8 * g + 2]) * inv, __uint_as_float(v[8 * g + 3]) * inv);
              o.z = pack_bf16x2(__uint_as_float(v[8 * g + 4]) * inv, __uint_as_float(v[8 * g + 5]) * inv);
              o.w = pack_bf16x2(__uint_as_float(v[8 * g + 6]) * inv, __uint_as_float(v[8 * g + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = o;
            }
          }
        }
        if (live) {
          const float m_nat = (m_used == -INFINITY) ? 0.f : m_used * (kSoftcap ? 1.f : p.scale);
          lse[static_cast<size_t>(head) * p.total + row] = l > 0.f ? m_nat + __logf(l) : 0.f;
        }
      }
    }
  }

  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);   // let copies in flight land
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ================================================================== backward
template <int D>
struct BwdCfg {
  static constexpr int kChunks = D / 64;
  static constexpr int kChunkBytes = kTile * 128;
  static constexpr int kTileBytes = kChunks * kChunkBytes;
  static constexpr int kRing = 3;                               // stages 0 / 1: Q of even / odd query tiles; stage 2: dO
  static constexpr int kDsBytes = 2 * kChunkBytes;              // dS^T: 128 key rows x 128 query columns
  static constexpr int kVecBytes = 8 * 2 * 64 * 4;              // lse, delta of a warp's 64 query columns, one copy per warp
  static constexpr int kDrainBytes = 4 * 4096;                  // one 32 x 32 fp32 staging piece per drain warp
  static constexpr int kSmemBytes = (2 + kRing) * kTileBytes + kDsBytes + kVecBytes + kDrainBytes + 1024;
  static constexpr int kThreads = 512;
  // registers per thread after the warpgroups have traded them (512 threads start with 128 each):
  // producer / MMA / allocator warps, the two element-wise warpgroups, the dQ drain warpgroup
  // How dQ leaves the drain warps. false: through a shared-memory staging piece as TMA reduce-add (whole
  // 128-byte lines). true: as vector reductions from registers (`red.global.add.v2.f32`, a quad of lanes
  // per 32-byte sector), which takes the staging round trip out of the shared-memory traffic that bounds
  // the loop, but measured slower (3.30 against 2.59 ms on 8 x 4096 x 24 / 8 heads x 128): the 64
  // reductions per thread and query tile hold up the load / store pipe, and step 2's stores behind them.
  static constexpr bool kDqRed = false;
  static constexpr int kRegsLight = 64, kRegsElem = 144, kRegsDrain = 160;
  static_assert(kRegsLight + 2 * kRegsElem + kRegsDrain == 4 * 128, "the register file must add up");
  static constexpr int kTmemCols = 512;
  static constexpr int kPCol = 32;                              // P^T (64 columns of bf16 pairs) inside S^T's columns:
                                                                // each warpgroup overwrites only columns it has read itself
  static constexpr int kDpCol = 128;                            // dP^T, later the dQ tile
  static constexpr int kDkCol = 256;
  static constexpr int kDvCol = 256 + D;
};

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (token, head)
template <int D>
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  float* __restrict__ delta, int total, int heads) {
  const long n = static_cast<long>(total) * heads;
  const int lane = threadIdx.x & 31;
  for (long w = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; w < n;
       w += (static_cast<long>(gridDim.x) * blockDim.x) >> 5) {
    const __nv_bfloat16* a = o + w * D;
    const __nv_bfloat16* b = d_o + w * D;
    float acc = 0.f;
    // D / 32 consecutive elements per lane
    constexpr int kPer = D / 32;
    const __nv_bfloat16* pa = a + lane * kPer;
    const __nv_bfloat16* pb = b + lane * kPer;
#pragma unroll
    for (int i = 0; i < kPer; i += 2) {
      const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(pa + i));
      const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(pb + i));
      acc = fmaf(x.x, y.x, acc);
      acc = fmaf(x.y, y.y, acc);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) {
      const long tok = w / heads;
      const int h = static_cast<int>(w - tok * heads);
      delta[static_cast<size_t>(h) * total + tok] = acc;
    }
  }
}

// Last pass over dQ: the fp32 accumulator becomes bf16, is rotated back (the inverse of the RoPE
// that was applied to q in place, when tables are given) and lands at its place in the caller's
// gradient tensor, whose tokens may be `dst_stride` elements apart (a slot of a packed qkv
// gradient). One thread per 8 elements; the interleaved layout pairs neighbours, the half layout
// pairs element i with i + rot_dim / 2.
struct DqFinish {
  const float* cos;
  const float* sin;
  const void* positions;
  int pos_is_i64;
  int rot_dim;          // 0: no rotation
  int interleaved;
};

template <int D>
__global__ void attn_dq_finish_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dst, long dst_stride,
                                      int total, int heads, DqFinish f) {
  constexpr int kVec = D / 8;
  const long n = static_cast<long>(total) * heads * kVec;
  const int half = f.rot_dim >> 1;
  for (long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < n;
       idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(idx % kVec);
    const long th = idx / kVec;
    const int h = static_cast<int>(th % heads);
    const long t = th / heads;
    const float* a = acc + (t * heads + h) * D;
    __nv_bfloat16* d = dst + t * dst_stride + h * D;
    auto load8 = [&](int e0, float (&v)[8]) {
      const float4 x = *reinterpret_cast<const float4*>(a + e0);
      const float4 y = *reinterpret_cast<const float4*>(a + e0 + 4);
      v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
    };
    auto store8 = [&](int e0, const float (&v)[8]) {
      uint4 o;
      o.x = pack_bf16x2(v[0], v[1]);
      o.y = pack_bf16x2(v[2], v[3]);
      o.z = pack_bf16x2(v[4], v[5]);
      o.w = pack_bf16x2(v[6], v[7]);
      *reinterpret_cast<uint4*>(d + e0) = o;
    };
    float v[8];
    if (8 * j >= f.rot_dim) {
      load8(8 * j, v);
      store8(8 * j, v);
      continue;
    }
    const long p = f.pos_is_i64 ? static_cast<long>(static_cast<const int64_t*>(f.positions)[t])
                                : static_cast<long>(static_cast<const int32_t*>(f.positions)[t]);
    if (f.interleaved) {
      load8(8 * j, v);
      const float4 c = *reinterpret_cast<const float4*>(f.cos + p * half + 4 * j);
      const float4 sn = *reinterpret_cast<const float4*>(f.sin + p * half + 4 * j);
      const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
      float o[8];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        o[2 * k] = v[2 * k] * cc[k] + v[2 * k + 1] * ss[k];
        o[2 * k + 1] = v[2 * k + 1] * cc[k] - v[2 * k] * ss[k];
      }
      store8(8 * j, o);
    } else {
      if (8 * j >= half) continue;            // written by the thread that owns the first half
      float hi[8], cc[8], ss[8], olo[8], ohi[8];
      load8(8 * j, v);
      load8(8 * j + half, hi);
      *reinterpret_cast<float4*>(cc) = *reinterpret_cast<const float4*>(f.cos + p * half + 8 * j);
      *reinterpret_cast<float4*>(cc + 4) = *reinterpret_cast<const float4*>(f.cos + p * half + 8 * j + 4);
      *reinterpret_cast<float4*>(ss) = *reinterpret_cast<const float4*>(f.sin + p * half + 8 * j);
      *reinterpret_cast<float4*>(ss + 4) = *reinterpret_cast<const float4*>(f.sin + p * half + 8 * j + 4);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        olo[k] = v[k] * cc[k] + hi[k] * ss[k];
        ohi[k] = hi[k] * cc[k] - v[k] * ss[k];
      }
      store8(8 * j, olo);
      store8(8 * j + half, ohi);
    }
  }
}

// Cycle counters of the backward kernel's roles (compiled in with -DHB_ATTN_PROFILE or a define in
// attention.h; read with attention_profile_read). Slot: 0 query tiles; MMA thread waits 1 dO ring,
// 2 dq_free, 3 p_ready, 4 Q ring, 5 ds_ready, 6 its loop; element-wise warp 4 lane 0: 7 wait dP, 8 wait S,
// 9 step 1 work, 10 step 2 work, 11 its loop; drain warp 12 lane 0: 12 wait dQ, 13 waits for the
// reduce engine, 14 its loop, 15 TMEM loads.
#ifdef HB_ATTN_PROFILE
__device__ unsigned long long hb_attn_prof[32];
// counters live in registers and reach memory once per CTA and role (an atomic per wait slowed the
// kernel threefold)
#define HB_PROF_DECL() long long _pacc[6] = {0, 0, 0, 0, 0, 0}
#define HB_PROF_BEGIN(t) const long long t = clock64()
#define HB_PROF_END(t, k) _pacc[k] += clock64() - (t)
#define HB_PROF_FLUSH(base, n, on)                                                                   \
  do {                                                                                                \
    if (on)                                                                                           \
      for (int _i = 0; _i < (n); ++_i)                                                                \
        atomicAdd(&hb_attn_prof[(base) + _i], static_cast<unsigned long long>(_pacc[_i]));            \
  } while (0)
#else
#define HB_PROF_DECL() do {} while (0)
#define HB_PROF_BEGIN(t) do {} while (0)
#define HB_PROF_END(t, k) do {} while (0)
#define HB_PROF_FLUSH(base, n, on) do {} while (0)
#endif

template <int D, bool kSoftcap>
__global__ void __launch_bounds__(512, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                const __grid_constant__ CUtensorMap tm_dq, float* __restrict__ dq_accum,
                const float* __restrict__ lse,
                const float* __restrict__ delta, __nv_bfloat16* __restrict__ dk, long dk_stride,
                __nv_bfloat16* __restrict__ dv, long dv_stride, const __grid_constant__ AttnParams p) {
  using C = BwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_kv_full;
  __shared__ __align__(8) uint64_t bar_ring_full[C::kRing];
  __shared__ __align__(8) uint64_t bar_ring_empty[C::kRing];
  __shared__ __align__(8) uint64_t bar_s_full, bar_dp_full, bar_p_ready, bar_ds_ready, bar_dq_full, bar_dq_free,
      bar_dkv_full;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  if (threadIdx.x == 0) abort_flag = p.status ? *reinterpret_cast<volatile int*>(p.status) : 0;
  __syncthreads();
  if (abort_flag) return;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t k_smem = smem_base;
  const uint32_t v_smem = smem_base + C::kTileBytes;
  const uint32_t ring = smem_base + 2 * C::kTileBytes;
  const uint32_t ds_smem = ring + C::kRing * C::kTileBytes;
  float* vec = reinterpret_cast<float*>(smem_raw + (ds_smem + C::kDsBytes - smem_u32(smem_raw)));
  const uint32_t drain_smem = ds_smem + C::kDsBytes + C::kVecBytes;
  // vec layout: [warp][lse2 | delta][64]: each elementwise warp stages its own copy, so the
  // eight warps never wait for one another
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int Hk = p.n_kv_heads, G = p.n_heads / Hk;
  int jk, hk;
  {
    const int id = blockIdx.x;
    if (!p.seg_start && p.seq_len % kTile == 0 && p.total % p.seq_len == 0) {
      const int per_seq = p.seq_len / kTile, nseq = p.total / p.seq_len;
      const int pos = id / (nseq * Hk);          // early key tiles are seen by the most queries: first
      const int rem = id % (nseq * Hk);
      jk = (rem / Hk) * per_seq + pos;
      hk = rem % Hk;
    } else {
      jk = id / Hk;
      hk = id % Hk;
    }
  }
  const int k0 = jk * kTile;
  int ib, ie;
  {
    int lo, hi, lo2, hi2;
    key_bounds(p, k0, lo, hi2);
    key_bounds(p, min(k0 + kTile - 1, p.total - 1), lo2, hi);
    ib = lo / kTile;
    ie = hi / kTile + 1;
    if (ie < ib) ie = ib;
  }
  const int n_i = ie - ib;
  const int n_it = n_i * G;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar_kv_full), 1);
    for (int s = 0; s < C::kRing; ++s) {
      mbar_init(smem_u32(&bar_ring_full[s]), 1);
      mbar_init(smem_u32(&bar_ring_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_s_full), 1);
    mbar_init(smem_u32(&bar_dp_full), 1);
    mbar_init(smem_u32(&bar_p_ready), 8);
    mbar_init(smem_u32(&bar_ds_ready), 8);
    mbar_init(smem_u32(&bar_dq_full), 1);
    mbar_init(smem_u32(&bar_dq_free), 4);
    mbar_init(smem_u32(&bar_dkv_full), 1);
    fence_barrier_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&tm_dq);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  // The four warpgroups trade registers, each at the top of its own branch (so that the code below
  // it is compiled for that budget): the light one (producer, MMA issuer, allocator) gives some up
  // and nobody else does, so the requests of the other three always find them.
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::kRegsLight));
  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ producer
    {
      const uint32_t full = smem_u32(&bar_kv_full);
      mbar_expect_tx(full, 2 * C::kTileBytes);
#pragma unroll
      for (int c = 0; c < C::kChunks; ++c) {
        tma_load_3d(k_smem + c * C::kChunkBytes, &tm_k, full, c * 64, hk, k0);
        tma_load_3d(v_smem + c * C::kChunkBytes, &tm_v, full, c * 64, hk, k0);
      }
    }
    // Q(it) lives from S(it) to dK(it), a whole query tile and a half, so it alternates between two
    // stages; dO(it) is done after dV(it), in the middle of its tile, and has the third stage to
    // itself. Either way a load is issued half a query tile or more before its first use.
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const int h = hk * G + it / n_i;
      const int q0 = (ib + it % n_i) * kTile;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const int stage = which == 0 ? (it & 1) : 2;
        const uint32_t phase = which == 0 ? ((it >> 1) & 1) : (it & 1);
        ok = mbar_wait(smem_u32(&bar_ring_empty[stage]), phase ^ 1, &abort_flag, p.status, kTimeoutEmpty);
        if (!ok) break;
        const uint32_t full = smem_u32(&bar_ring_full[stage]);
        mbar_expect_tx(full, C::kTileBytes);
        const uint32_t dst = ring + stage * C::kTileBytes;
#pragma unroll
        for (int c = 0; c < C::kChunks; ++c)
          tma_load_3d(dst + c * C::kChunkBytes, which == 0 ? &tm_q : &tm_do, full, c * 64, h, q0);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------ MMA issuer
    // Order per query tile: dP(it), dV(it), S(it + 1), dK(it), dQ(it). S of the next tile is issued
    // as soon as dV has consumed P, so the elementwise warps can turn it into P(it + 1) while the
    // tensor cores run dK(it) and dQ(it).
    constexpr uint32_t idesc_kk = make_idesc_bf16(kTile, kTile, false, false);   // S^T, dP^T
    constexpr uint32_t idesc_acc = make_idesc_bf16(kTile, D, false, true);       // dV, dK
    constexpr uint32_t idesc_dq = make_idesc_bf16(kTile, D, true, true);         // dQ
    HB_PROF_DECL();
    bool ok = mbar_wait(smem_u32(&bar_kv_full), 0, &abort_flag, p.status, kTimeoutFull);
    const uint32_t k_lo = desc_lo(k_smem, 0), v_lo = desc_lo(v_smem, 0);
    const uint32_t k_mn_lo = desc_lo(k_smem, C::kChunkBytes), ds_lo = desc_lo(ds_smem, 0),
                   ds_mn_lo = desc_lo(ds_smem, C::kChunkBytes);
    auto issue_s = [&](int it) -> bool {
      HB_PROF_BEGIN(tq);
      if (!mbar_wait(smem_u32(&bar_ring_full[it & 1]), (it >> 1) & 1, &abort_flag, p.status, kTimeoutFull))
        return false;
      HB_PROF_END(tq, 3);
      tc_fence_after();
      const uint32_t q_lo = desc_lo(ring + (it & 1) * C::kTileBytes, 0);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t off = static_cast<uint32_t>(((ks >> 2) * C::kChunkBytes + (ks & 3) * 32) >> 4);
        umma_ss(tmem_base, k_lo + off, q_lo + off, idesc_kk, ks != 0);
      }
      umma_commit(smem_u32(&bar_s_full));
      return true;
    };
    if (ok && n_it > 0) ok = issue_s(0);
    HB_PROF_BEGIN(tloop);
    for (int it = 0; it < n_it && ok; ++it) {
      const uint32_t q_addr = ring + (it & 1) * C::kTileBytes;
      const uint32_t o_addr = ring + 2 * C::kTileBytes;
      const uint32_t par = it & 1;
      // dP^T = V dO^T (its columns held the previous dQ tile until the drain finished)
      HB_PROF_BEGIN(t1);
      ok = mbar_wait(smem_u32(&bar_ring_full[2]), it & 1, &abort_flag, p.status, kTimeoutFull);
      HB_PROF_END(t1, 0);
      HB_PROF_BEGIN(t2);
      if (ok && it > 0)
        ok = mbar_wait(smem_u32(&bar_dq_free), (it - 1) & 1, &abort_flag, p.status, kTimeoutTmemEmpty);
      HB_PROF_END(t2, 1);
      if (!ok) break;
      tc_fence_after();
      const uint32_t o_lo = desc_lo(o_addr, 0), o_mn_lo = desc_lo(o_addr, C::kChunkBytes);
      const uint32_t q_mn_lo = desc_lo(q_addr, C::kChunkBytes);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t off = static_cast<uint32_t>(((ks >> 2) * C::kChunkBytes + (ks & 3) * 32) >> 4);
        umma_ss(tmem_base + C::kDpCol, v_lo + off, o_lo + off, idesc_kk, ks != 0);
      }
      umma_commit(smem_u32(&bar_dp_full));
      // dV += P^T dO
      HB_PROF_BEGIN(t3);
      ok = mbar_wait(smem_u32(&bar_p_ready), par, &abort_flag, p.status, kTimeoutTmemEmpty);
      HB_PROF_END(t3, 2);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < kTile / 16; ++ks)
        umma_ts(tmem_base + C::kDvCol, tmem_base + C::kPCol + ks * 8, o_mn_lo + static_cast<uint32_t>((ks * 2048) >> 4),
                idesc_acc, it > 0 || ks != 0);
      umma_commit(smem_u32(&bar_ring_empty[2]));
      // S^T of the next tile, over the P that dV has just been issued on (the tensor cores run
      // one CTA's instructions in issue order)
      if (it + 1 < n_it) {
        ok = issue_s(it + 1);
        if (!ok) break;
      }
      // dK += dS^T Q, dQ = dS K
      HB_PROF_BEGIN(t5);
      ok = mbar_wait(smem_u32(&bar_ds_ready), par, &abort_flag, p.status, kTimeoutTmemEmpty);
      HB_PROF_END(t5, 4);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < kTile / 16; ++ks) {
        const uint32_t a_off = static_cast<uint32_t>(((ks >> 2) * C::kChunkBytes + (ks & 3) * 32) >> 4);
        umma_ss(tmem_base + C::kDkCol, ds_lo + a_off, q_mn_lo + static_cast<uint32_t>((ks * 2048) >> 4), idesc_acc,
                it > 0 || ks != 0);
      }
#pragma unroll
      for (int ks = 0; ks < kTile / 16; ++ks)
        umma_ss(tmem_base + C::kDpCol, ds_mn_lo + static_cast<uint32_t>((ks * 2048) >> 4),
                k_mn_lo + static_cast<uint32_t>((ks * 2048) >> 4), idesc_dq, ks != 0);
      umma_commit(smem_u32(&bar_dq_full));
      umma_commit(smem_u32(&bar_ring_empty[it & 1]));
    }
    HB_PROF_END(tloop, 5);
    HB_PROF_FLUSH(1, 6, true);
#ifdef HB_ATTN_PROFILE
    atomicAdd(&hb_attn_prof[0], static_cast<unsigned long long>(n_it));
#endif
    if (ok) umma_commit(smem_u32(&bar_dkv_full));
  }
  } else if (warp < 12) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::kRegsElem));
    // ------------------------------------------------------------ elementwise
    // Two warpgroups share every 128 x 128 tile: warps 4-7 take query columns 0-63 of each key
    // row, warps 8-11 columns 64-127 (a warp reads the TMEM lane quarter warp % 4). Per query
    // tile: P (step 1) and dS (step 2); step 1 of the next tile runs under the dK / dQ products of
    // this one. The dQ tile leaves through the drain warpgroup (warps 12-15). With soft-capping
    // step 1 parks a factor in the dS buffer, so it first waits until dK / dQ have read dS.
    const int wg = (warp - 4) >> 2;            // which half of the columns
    const int wq = warp & 3;
    const int r = wq * 32 + lane;              // key row in steps 1 and 2, query row in the drain
    const int kpos = k0 + r;
    int qlo, qhi;
    key_bounds(p, kpos, qlo, qhi);
    const uint32_t lane_addr = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_addr + wg * 64;                 // this half of S^T
    const uint32_t p_addr = tmem_base + lane_addr + C::kPCol + wg * 32;      // this half of P^T (bf16 pairs)
    const uint32_t dp_addr = tmem_base + C::kDpCol + lane_addr + wg * 64;    // this half of dP^T
    const float c2 = kSoftcap ? kLog2e : p.scale * kLog2e;
    const float cap_in = kSoftcap ? p.scale / p.softcap : 0.f;
    // this thread's 64 columns of dS^T are one 128-byte row of the buffer's half `wg`
    const uint32_t ds_row = ds_smem + wg * C::kChunkBytes + r * 128;
    float* lse2 = vec + (warp - 4) * 2 * 64;
    float* dlt = lse2 + 64;
    uint32_t pk[32];
    bool ok = true;
    float pre[4], nxt[4];
    HB_PROF_DECL();

    // lse / delta of this warp's 64 query columns: fetched two query tiles ahead into registers (the
    // loads compete with the tile loads and the dQ reductions for L2), parked in shared memory
    // right before use
    auto fetch_vectors = [&](int it, float (&dst)[4]) {
      const int h = hk * G + it / n_i;
      const int q0 = (ib + it % n_i) * kTile + wg * 64;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int q = q0 + lane + 32 * u;
        const bool live = q < p.total;
        // plain predicated loads: nothing here may depend on the loaded values, or the warp would sit
        // on the load's latency right here instead of at the park two tiles later
        dst[u] = INFINITY;
        dst[2 + u] = 0.f;
        if (live) {
          dst[u] = __ldg(lse + static_cast<size_t>(h) * p.total + q);
          dst[2 + u] = __ldg(delta + static_cast<size_t>(h) * p.total + q);
        }
      }
    };
    auto park_vectors = [&]() {
      __syncwarp();                 // every lane is done with the previous tile's values
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        lse2[lane + 32 * u] = pre[u] * kLog2e;
        dlt[lane + 32 * u] = pre[2 + u];
      }
      __syncwarp();
    };
    // ---- step 1: P^T = exp2(S^T c2 - lse) as bf16 pairs, into TMEM and into `pk`
    auto step1 = [&](int it) -> bool {
      const int q0 = (ib + it % n_i) * kTile + wg * 64;
      const bool mask_tile = __any_sync(0xffffffffu, q0 < qlo || q0 + 63 > qhi);
      HB_PROF_BEGIN(tw);
      bool good = mbar_wait(smem_u32(&bar_s_full), it & 1, &abort_flag, p.status, kTimeoutTmemFull);
      good = __all_sync(0xffffffffu, good);
      HB_PROF_END(tw, 1);
      if (!good) return false;
      HB_PROF_BEGIN(tk);
      tc_fence_after();
      uint32_t v[2][32];
      tmem_ld_32x32(s_addr, v[0]);
      tmem_ld_32x32(s_addr + 32, v[1]);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float pr[32];
#pragma unroll
        for (int i4 = 0; i4 < 8; ++i4) {
          const float4 l4 = *reinterpret_cast<const float4*>(lse2 + c * 32 + i4 * 4);
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int i = i4 * 4 + u;
            float s = __uint_as_float(v[c][i]);
            if (kSoftcap) {
              const float th = tanh_fast(s * cap_in);
              s = p.softcap * th;
              v[c][i] = __float_as_uint(1.f - th * th);
            }
            pr[i] = ex2_fast(fmaf(s, c2, -ls[u]));
          }
        }
        if (mask_tile) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int q = q0 + c * 32 + i;
            if (q < qlo || q > qhi) pr[i] = 0.f;
          }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[c * 16 + i] = pack_bf16x2(pr[2 * i], pr[2 * i + 1]);
        if (kSoftcap) {
          // park d(capped score)/d(score) in this row's slot of the dS buffer until dP arrives
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const uint32_t u = static_cast<uint32_t>(c * 4 + g);
            st_shared_v4(ds_row + ((u ^ (r & 7)) << 4),
                         pack_bf16x2(__uint_as_float(v[c][8 * g]), __uint_as_float(v[c][8 * g + 1])),
                         pack_bf16x2(__uint_as_float(v[c][8 * g + 2]), __uint_as_float(v[c][8 * g + 3])),
                         pack_bf16x2(__uint_as_float(v[c][8 * g + 4]), __uint_as_float(v[c][8 * g + 5])),
                         pack_bf16x2(__uint_as_float(v[c][8 * g + 6]), __uint_as_float(v[c][8 * g + 7])));
          }
        }
      }
      // both of this thread's S chunks are in registers: P may now overwrite S's columns
      tmem_st_32x32(p_addr, pk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_p_ready));
      HB_PROF_END(tk, 2);
      return true;
    };
    // ---- step 2: dS^T = P^T (dP^T - delta) scale, bf16, into shared memory
    auto step2 = [&](int it) -> bool {
      HB_PROF_BEGIN(tw);
      bool good = mbar_wait(smem_u32(&bar_dp_full), it & 1, &abort_flag, p.status, kTimeoutTmemFull);
      good = __all_sync(0xffffffffu, good);
      HB_PROF_END(tw, 0);
      if (!good) return false;
      HB_PROF_BEGIN(tk);
      tc_fence_after();
      uint32_t v[2][32];
      tmem_ld_32x32(dp_addr, v[0]);
      tmem_ld_32x32(dp_addr + 32, v[1]);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float ds[32];
#pragma unroll
        for (int i4 = 0; i4 < 8; ++i4) {
          const float4 d4 = *reinterpret_cast<const float4*>(dlt + c * 32 + i4 * 4);
          const float2 p0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk[c * 16 + i4 * 2]));
          const float2 p1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk[c * 16 + i4 * 2 + 1]));
          ds[i4 * 4] = p0.x * p.scale * (__uint_as_float(v[c][i4 * 4]) - d4.x);
          ds[i4 * 4 + 1] = p0.y * p.scale * (__uint_as_float(v[c][i4 * 4 + 1]) - d4.y);
          ds[i4 * 4 + 2] = p1.x * p.scale * (__uint_as_float(v[c][i4 * 4 + 2]) - d4.z);
          ds[i4 * 4 + 3] = p1.y * p.scale * (__uint_as_float(v[c][i4 * 4 + 3]) - d4.w);
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint32_t u = static_cast<uint32_t>(c * 4 + g);
          const uint32_t addr = ds_row + ((u ^ (r & 7)) << 4);
          if (kSoftcap) {
            const uint4 gq = ld_shared_v4(addr);
            const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gq);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 gg = __bfloat1622float2(g2[i]);
              ds[8 * g + 2 * i] *= gg.x;
              ds[8 * g + 2 * i + 1] *= gg.y;
            }
          }
          st_shared_v4(addr, pack_bf16x2(ds[8 * g], ds[8 * g + 1]), pack_bf16x2(ds[8 * g + 2], ds[8 * g + 3]),
                       pack_bf16x2(ds[8 * g + 4], ds[8 * g + 5]), pack_bf16x2(ds[8 * g + 6], ds[8 * g + 7]));
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();      // the tensor cores read dS^T through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_ds_ready));
      HB_PROF_END(tk, 3);
      return true;
    };
    if (n_it > 0) {
      fetch_vectors(0, pre);
      park_vectors();
      if (n_it > 1) fetch_vectors(1, pre);
      ok = step1(0);
    }
    HB_PROF_BEGIN(tloop);
    for (int it = 0; it < n_it && ok; ++it) {
      const bool more = it + 1 < n_it;
      if (it + 2 < n_it) fetch_vectors(it + 2, nxt);
      ok = step2(it);
      if (!ok) break;
      if (more) {
        if (kSoftcap) {
          // the factor goes into the dS rows: dK(it) and dQ(it) must have read dS(it)
          ok = mbar_wait(smem_u32(&bar_dq_full), it & 1, &abort_flag, p.status, kTimeoutTmemFull);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        park_vectors();
#pragma unroll
        for (int u = 0; u < 4; ++u) pre[u] = nxt[u];
        ok = step1(it + 1);
      }
    }
    HB_PROF_END(tloop, 4);
    HB_PROF_FLUSH(7, 5, warp == 4 && lane == 0);
    // ---- dK, dV of this key tile: the first warpgroup writes dK, the second dV
    if (ok && n_it > 0) {
      ok = mbar_wait(smem_u32(&bar_dkv_full), 0, &abort_flag, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      // (all 32 lanes stay together here: tcgen05.ld is a warp-wide instruction; only the stores
      // below depend on whether this lane's key row exists)
      const bool live = kpos < p.total;
      if (n_it > 0) tc_fence_after();
      const uint32_t addr = tmem_base + (wg == 0 ? C::kDkCol : C::kDvCol) + lane_addr;
      __nv_bfloat16* dst = wg == 0 ? dk + static_cast<size_t>(kpos) * dk_stride + hk * D
                                   : dv + static_cast<size_t>(kpos) * dv_stride + hk * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        if (n_it > 0) {
          tmem_ld_32x32(addr + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;       // no query sees these keys
        }
        if (live) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[8 * g]), __uint_as_float(v[8 * g + 1]));
            o.y = pack_bf16x2(__uint_as_float(v[8 * g + 2]), __uint_as_float(v[8 * g + 3]));
            o.z = pack_bf16x2(__uint_as_float(v[8 * g + 4]), __uint_as_float(v[8 * g + 5]));
            o.w = pack_bf16x2(__uint_as_float(v[8 * g + 6]), __uint_as_float(v[8 * g + 7]));
            *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = o;
          }
        }
      }
    }
  }

  else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::kRegsDrain));
    // ------------------------------------------------------------ dQ drain
    // dQ(it) = dS K sits in the columns that take dP of the next query tile. Each warp reads its 32
    // query rows (all D columns) into registers, frees the columns, and adds the rows into dq_accum:
    // as vector reductions from registers, or (kDqRed false) 32 columns at a time through its
    // staging piece as bulk tensor reductions.
    const int wq = warp & 3;
    const uint32_t dq_addr = tmem_base + C::kDpCol + (static_cast<uint32_t>(wq * 32) << 16);
    const uint32_t piece = drain_smem + wq * 4096;
    bool ok = true;
    bool reads_pending = false;
    HB_PROF_DECL();
    HB_PROF_BEGIN(tloop);
    for (int it = 0; it < n_it && ok; ++it) {
      const int h = hk * G + it / n_i;
      const int q0 = (ib + it % n_i) * kTile;
      HB_PROF_BEGIN(tw);
      ok = mbar_wait(smem_u32(&bar_dq_full), it & 1, &abort_flag, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      HB_PROF_END(tw, 0);
      if (!ok) break;
      HB_PROF_BEGIN(tl);
      tc_fence_after();
      if constexpr (C::kDqRed) {
        // rows wq * 32 + {0..15} and + {16..31} of the tile, D columns in blocks of 32
        uint32_t v[2 * (D / 32)][16];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
#pragma unroll
          for (int cg = 0; cg < D / 32; ++cg)
            tmem_ld_16x256b_x4(dq_addr + (static_cast<uint32_t>(hh * 16) << 16) + cg * 32, v[hh * (D / 32) + cg]);
        tmem_ld_wait();
        // the tile is in registers: its TMEM columns can take the next dP^T already
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_dq_free));
        HB_PROF_END(tl, 3);
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int row = q0 + wq * 32 + hh * 16 + half * 8 + (lane >> 2);
            if (row < p.total) {
              float* dst = dq_accum + (static_cast<size_t>(row) * p.n_heads + h) * D + 2 * (lane & 3);
#pragma unroll
              for (int cg = 0; cg < D / 32; ++cg)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  red_add_v2_f32(dst + cg * 32 + j * 8, v[hh * (D / 32) + cg][4 * j + 2 * half],
                                 v[hh * (D / 32) + cg][4 * j + 2 * half + 1]);
            }
          }
        }
      } else {
        uint32_t v[D / 32][32];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tmem_ld_32x32(dq_addr + c * 32, v[c]);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_dq_free));
        HB_PROF_END(tl, 3);
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          if (reads_pending) {
            // the piece may only be rewritten once the reduction that reads it has done so
            HB_PROF_BEGIN(tr);
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            __syncwarp();
            HB_PROF_END(tr, 1);
          }
#pragma unroll
          for (int g = 0; g < 8; ++g)
            st_shared_v4(piece + lane * 128 + ((static_cast<uint32_t>(g) ^ (lane & 7)) << 4), v[c][4 * g],
                         v[c][4 * g + 1], v[c][4 * g + 2], v[c][4 * g + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            asm volatile(
                "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                    reinterpret_cast<uint64_t>(&tm_dq)),
                "r"(piece), "r"(c * 32), "r"(h), "r"(q0 + wq * 32)
                : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          reads_pending = true;
        }
      }
    }
    HB_PROF_END(tloop, 2);
    HB_PROF_FLUSH(12, 4, warp == 12 && lane == 0);
    // every reduction this lane issued has to land before the CTA's shared memory goes away
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    __syncwarp();
  }

  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ================================================================== host side
#ifdef HB_ATTN_PROFILE
}  // namespace
cudaError_t attention_profile_read(unsigned long long* out32, bool reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out32, hb_attn_prof, sizeof(unsigned long long) * 32);
  if (e != cudaSuccess || !reset) return e;
  unsigned long long zeros[32] = {};
  return cudaMemcpyToSymbol(hb_attn_prof, zeros, sizeof(zeros));
}
namespace {
#endif
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(ptr);
  return fn;
}

// [tokens, heads, head_dim] bf16 with `tok_stride` elements between tokens; box = 128 tokens of
// one head, 64 elements wide, 128-byte swizzle, zeros beyond the last token.
bool make_tmap_heads(CUtensorMap* map, const void* base, int tokens, int heads, int head_dim, long tok_stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    // the encode call is a driver entry point: bind the primary context in threads that have not
    // made a runtime call yet (autograd's backward workers)
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return false;
    (void)cudaFree(nullptr);
    ctx_bound = true;
  }
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(heads),
                        static_cast<cuuint64_t>(tokens)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_dim) * 2, static_cast<cuuint64_t>(tok_stride) * 2};
  cuuint32_t box[3] = {64, 1, kTile};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "halite_b200: attention tensor map failed (%d): tokens=%d heads=%d dim=%d stride=%ld base=%p\n",
            static_cast<int>(r), tokens, heads, head_dim, tok_stride, base);
  return r == CUDA_SUCCESS;
}

// fp32 [tokens, heads, head_dim] contiguous; box = 32 tokens of one head, 32 columns (128 bytes),
// 128-byte swizzle: the destination of the dQ reductions.
bool make_tmap_dq(CUtensorMap* map, void* base, int tokens, int heads, int head_dim) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(heads),
                        static_cast<cuuint64_t>(tokens)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_dim) * 4, static_cast<cuuint64_t>(heads) * head_dim * 4};
  cuuint32_t box[3] = {32, 1, 32};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "halite_b200: dq tensor map failed (%d): tokens=%d heads=%d dim=%d base=%p\n",
            static_cast<int>(r), tokens, heads, head_dim, base);
  return r == CUDA_SUCCESS;
}

cudaError_t check_args(const AttnArgs& a) {
  if (a.total <= 0) return cudaSuccess;
  if ((a.head_dim != 64 && a.head_dim != 128) || a.n_heads <= 0 || a.n_kv_heads <= 0 ||
      a.n_heads % a.n_kv_heads != 0)
    return cudaErrorInvalidValue;
  if (!a.seg_start && a.seq_len <= 0) return cudaErrorInvalidValue;
  if ((a.seg_start == nullptr) != (a.seg_end == nullptr)) return cudaErrorInvalidValue;
  if (a.q_tok_stride % 8 || a.k_tok_stride % 8 || a.v_tok_stride % 8) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v)) & 15)
    return cudaErrorInvalidValue;
  return cudaSuccess;
}

AttnParams to_params(const AttnArgs& a) {
  AttnParams p;
  p.total = a.total;
  p.n_heads = a.n_heads;
  p.n_kv_heads = a.n_kv_heads;
  p.seq_len = a.seq_len > 0 ? a.seq_len : a.total;
  p.seg_start = a.seg_start;
  p.seg_end = a.seg_end;
  p.causal = a.causal ? 1 : 0;
  p.window = a.window;
  p.scale = a.scale;
  p.softcap = a.softcap;
  p.status = a.status;
  return p;
}

template <int D, bool SC>
cudaError_t launch_fwd(const AttnArgs& a, void* out, float* lse) {
  using C = FwdCfg<D>;
  CUtensorMap tq, tk, tv;
  if (!make_tmap_heads(&tq, a.q, a.total, a.n_heads, D, a.q_tok_stride) ||
      !make_tmap_heads(&tk, a.k, a.total, a.n_kv_heads, D, a.k_tok_stride) ||
      !make_tmap_heads(&tv, a.v, a.total, a.n_kv_heads, D, a.v_tok_stride))
    return cudaErrorInvalidValue;
  auto kern = attn_fwd_kernel<D, SC>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const int nqb = (a.total + 255) / 256;
  kern<<<nqb * a.n_heads, C::kThreads, C::kSmemBytes, a.stream>>>(tq, tk, tv, static_cast<__nv_bfloat16*>(out), lse,
                                                                  to_params(a));
  return cudaGetLastError();
}

template <int D, bool SC>
cudaError_t launch_bwd(const AttnArgs& a, const void* o, const void* d_o, const float* lse, float* delta,
                       float* dq_accum, void* dq, long dq_stride, const AttnDqRotation& rot, void* dk, long dk_stride,
                       void* dv, long dv_stride) {
  using C = BwdCfg<D>;
  CUtensorMap tq, tk, tv, tdo, tdq;
  if (!make_tmap_heads(&tq, a.q, a.total, a.n_heads, D, a.q_tok_stride) ||
      !make_tmap_heads(&tk, a.k, a.total, a.n_kv_heads, D, a.k_tok_stride) ||
      !make_tmap_heads(&tv, a.v, a.total, a.n_kv_heads, D, a.v_tok_stride) ||
      !make_tmap_heads(&tdo, d_o, a.total, a.n_heads, D, static_cast<long>(a.n_heads) * D) ||
      !make_tmap_dq(&tdq, dq_accum, a.total, a.n_heads, D))
    return cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(dq_accum) & 15) return cudaErrorInvalidValue;
  auto kern = attn_bwd_kernel<D, SC>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const size_t n = static_cast<size_t>(a.total) * a.n_heads * D;
  cudaError_t e = cudaMemsetAsync(dq_accum, 0, n * sizeof(float), a.stream);
  if (e != cudaSuccess) return e;
  {
    const long warps = static_cast<long>(a.total) * a.n_heads;
    const int grid = static_cast<int>(std::min<long>((warps + 7) / 8, 148L * 16));
    attn_delta_kernel<D><<<grid, 256, 0, a.stream>>>(static_cast<const __nv_bfloat16*>(o),
                                                      static_cast<const __nv_bfloat16*>(d_o), delta, a.total,
                                                      a.n_heads);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  const int nkt = (a.total + kTile - 1) / kTile;
  kern<<<nkt * a.n_kv_heads, C::kThreads, C::kSmemBytes, a.stream>>>(
      tq, tk, tv, tdo, tdq, dq_accum, lse, delta, static_cast<__nv_bfloat16*>(dk), dk_stride,
      static_cast<__nv_bfloat16*>(dv), dv_stride, to_params(a));
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  {
    DqFinish f;
    f.cos = rot.cos;
    f.sin = rot.sin;
    f.positions = rot.positions;
    f.pos_is_i64 = rot.pos_is_i64 ? 1 : 0;
    f.rot_dim = (rot.cos && rot.sin && rot.positions) ? rot.rot_dim : 0;
    f.interleaved = rot.interleaved ? 1 : 0;
    const long nvec = static_cast<long>(n / 8);
    const int grid = static_cast<int>(std::min<long>((nvec + 255) / 256, 148L * 16));
    attn_dq_finish_kernel<D><<<grid, 256, 0, a.stream>>>(dq_accum, static_cast<__nv_bfloat16*>(dq), dq_stride, a.total,
                                                         a.n_heads, f);
    e = cudaGetLastError();
  }
  return e;
}

}  // namespace

cudaError_t attention_fwd(const AttnArgs& a, void* out, float* lse) {
  cudaError_t e = check_args(a);
  if (e != cudaSuccess || a.total <= 0) return e;
  const bool sc = a.softcap > 0.f;
  if (a.head_dim == 128) return sc ? launch_fwd<128, true>(a, out, lse) : launch_fwd<128, false>(a, out, lse);
  return sc ? launch_fwd<64, true>(a, out, lse) : launch_fwd<64, false>(a, out, lse);
}

cudaError_t attention_bwd(const AttnArgs& a, const void* o, const void* d_o, const float* lse, float* delta,
                          float* dq_accum, void* dq, long dq_tok_stride, const AttnDqRotation& rot, void* dk,
                          long dk_tok_stride, void* dv, long dv_tok_stride) {
  cudaError_t e = check_args(a);
  if (e != cudaSuccess || a.total <= 0) return e;
  if (dk_tok_stride % 8 || dv_tok_stride % 8 || dq_tok_stride % 8) return cudaErrorInvalidValue;
  if (rot.cos && (rot.rot_dim <= 0 || rot.rot_dim > a.head_dim || rot.rot_dim % (rot.interleaved ? 8 : 16)))
    return cudaErrorInvalidValue;
  const bool sc = a.softcap > 0.f;
#define HB_ATTN_BWD(DD, SS) \
  launch_bwd<DD, SS>(a, o, d_o, lse, delta, dq_accum, dq, dq_tok_stride, rot, dk, dk_tok_stride, dv, dv_tok_stride)
  if (a.head_dim == 128) return sc ? HB_ATTN_BWD(128, true) : HB_ATTN_BWD(128, false);
  return sc ? HB_ATTN_BWD(64, true) : HB_ATTN_BWD(64, false);
#undef HB_ATTN_BWD
}

}  // namespace hb
