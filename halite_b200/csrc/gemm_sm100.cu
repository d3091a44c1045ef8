// bf16 GEMM for sm_100a: D[M,N] = A (*) B with fp32 accumulation in tensor memory.
//
// One persistent CTA per SM, 256 threads, four roles:
//   warp 0 (one lane)  TMA producer: cp.async.bulk.tensor tiles -> 128B-swizzled smem ring
//   warp 1 (one lane)  MMA issuer:   tcgen05.mma kind::f16, 128 x BN x 16 per instruction,
//                                     accumulator double-buffered in TMEM (2 x BN columns)
//   warp 2             TMEM allocation / release
//   warps 4..7         epilogue: tcgen05.ld -> registers -> global (bf16 or fp32,
//                                 optional accumulate), overlapped with the next tile's MMAs
//
// Operand layouts (both bf16):
//   A "K-major"  : memory [M, K] row-major      A "MN-major": memory [K, M] row-major
//   B "K-major"  : memory [N, K] row-major      B "MN-major": memory [K, N] row-major
// so the three training GEMMs need no transposes:
//   forward  Y  = X W^T      : A K-major (X),   B K-major (W)
//   dgrad    dX = dY W       : A K-major (dY),  B MN-major (W  [N_out, K_in] = [K_gemm, N_gemm])
//   wgrad    dW = dY^T X     : A MN-major (dY), B MN-major (X)
//
// Replaces the cuBLAS calls behind every nn.Linear of the reference
// (configs/models/transformer.py:124-177,292).
#include <stdio.h>
#include <stdlib.h>

#include <mutex>
#include <vector>

#include "gemm.h"
#include "sm100.cuh"

namespace hb {

namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;   // 64 bf16 = one 128-byte swizzle row
constexpr int kUK = 16;   // K of one tcgen05.mma for 16-bit inputs
constexpr int kThreads = 256;
constexpr int kGroupM = 16;  // raster: kGroupM row-tiles share the same column sweep

template <int BN>
struct Cfg {
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128) ? 6 : 8;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingBytes = 4 * 32 * 128;  // per epilogue warp: 32 rows x 128 bytes
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024;  // +1024: alignment
  static constexpr int kTmemCols = 2 * BN;
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = kGroupM * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * kGroupM;
  const int gsz = min(kGroupM, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

template <typename OutT>
__device__ __forceinline__ void store_chunk(OutT* __restrict__ p, const uint32_t (&v)[32],
                                            int valid, bool vec_ok, bool accumulate);

template <>
__device__ __forceinline__ void store_chunk<__nv_bfloat16>(__nv_bfloat16* __restrict__ p,
                                                           const uint32_t (&v)[32], int valid,
                                                           bool vec_ok, bool accumulate) {
  if (valid == 32 && vec_ok) {
    uint4* p4 = reinterpret_cast<uint4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[i * 8 + j]);
      if (accumulate) {
        uint4 old = p4[i];
        const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 o = __bfloat1622float2(o2[j]);
          f[2 * j] += o.x;
          f[2 * j + 1] += o.y;
        }
      }
      uint4 out;
      out.x = pack_bf16x2(f[0], f[1]);
      out.y = pack_bf16x2(f[2], f[3]);
      out.z = pack_bf16x2(f[4], f[5]);
      out.w = pack_bf16x2(f[6], f[7]);
      p4[i] = out;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < valid) {
        float x = __uint_as_float(v[j]);
        if (accumulate) x += __bfloat162float(p[j]);
        p[j] = __float2bfloat16_rn(x);
      }
    }
  }
}

template <>
__device__ __forceinline__ void store_chunk<float>(float* __restrict__ p, const uint32_t (&v)[32],
                                                   int valid, bool vec_ok, bool accumulate) {
  if (valid == 32 && vec_ok) {
    float4* p4 = reinterpret_cast<float4*>(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float4 o = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                             __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
      if (accumulate) {
        float4 old = p4[i];
        o.x += old.x;
        o.y += old.y;
        o.z += old.z;
        o.w += old.w;
      }
      p4[i] = o;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < valid) {
        float x = __uint_as_float(v[j]);
        if (accumulate) x += p[j];
        p[j] = x;
      }
    }
  }
}

// ---- fused gather helpers ------------------------------------------------------------
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded spin until *flag >= want. `sys` selects system scope (flags written by other GPUs).
__device__ __forceinline__ bool wait_flag(const int* flag, int want, bool sys,
                                          volatile int* abort_flag, int* status) {
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    const int v = sys ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
    if (v >= want) return true;
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > kWaitBudgetNs) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, (int)kTimeoutPeerFlag);
        return false;
      }
    }
    __nanosleep(64);
  }
}

// Wait for the granules covering operand rows [row0, row0 + nrows) of the gathered buffer.
__device__ __forceinline__ bool wait_rows(const GatherParams& gp, long row0, long nrows, long total_rows,
                                          volatile int* abort_flag, int* status) {
  const long r1 = min(row0 + nrows, total_rows);
  if (r1 <= row0) return true;
  const long lo = gp.dep_base_offset + row0 * gp.dep_row_bytes;
  const long hi = gp.dep_base_offset + r1 * gp.dep_row_bytes - 1;
  const long total = gp.chunk_bytes * gp.n_chunks;
  if (hi < 0 || lo >= total) return true;
  // flags are numbered chunk by chunk (a chunk's last granule may be short), like the copy CTAs do
  const long gpc = (gp.chunk_bytes + gp.granule_bytes - 1) / gp.granule_bytes;
  const long b0 = max(lo, 0L), b1 = min(hi, total - 1);
  for (long c = b0 / gp.chunk_bytes; c <= b1 / gp.chunk_bytes; ++c) {
    const long base = c * gp.chunk_bytes;
    const long g0 = (max(b0, base) - base) / gp.granule_bytes;
    const long g1 = (min(b1, base + gp.chunk_bytes - 1) - base) / gp.granule_bytes;
    for (long g = g0; g <= g1; ++g)
      if (!wait_flag(gp.flags + c * gpc + g, gp.epoch, false, abort_flag, status)) return false;
  }
  return true;
}

// Body of a copy CTA: granules are dealt round-robin over the copy CTAs, in address order.
__device__ __forceinline__ void gather_copy_cta(const GatherParams& gp, int cta, volatile int* abort_flag,
                                                int* status) {
  const long gpc = (gp.chunk_bytes + gp.granule_bytes - 1) / gp.granule_bytes;  // granules per chunk
  const long n_gran = gpc * gp.n_chunks;
  __shared__ int s_ok;
  // Chunks are visited in the order the tiles consume them: the local chunk first (nothing to
  // copy, its flags go up at once), then the following ranks' chunks, so each GPU starts on a
  // different peer.
  for (long it = cta; it < n_gran; it += gp.n_copy_ctas) {
    const int chunk = static_cast<int>((it / gpc + gp.first_chunk) % gp.n_chunks);
    const long off = (it % gpc) * gp.granule_bytes;
    const long gi = chunk * gpc + it % gpc;
    const long bytes = min(gp.granule_bytes, gp.chunk_bytes - off);
    if (gp.src[chunk] != nullptr) {
      if (threadIdx.x == 0) {
        s_ok = 1;
        if (gp.ready && !wait_flag(gp.ready + chunk, gp.epoch, true, abort_flag, status)) s_ok = 0;
      }
      __syncthreads();
      if (s_ok) {
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(gp.src[chunk]) + off);
        uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(gp.dst_base) + chunk * gp.chunk_bytes + off);
        const long n16 = bytes >> 4;
        long i = threadIdx.x;
        for (; i + 3 * blockDim.x < n16; i += 4 * blockDim.x) {
          const uint4 a = src[i], b = src[i + blockDim.x], c = src[i + 2 * blockDim.x],
                      d = src[i + 3 * blockDim.x];
          dst[i] = a;
          dst[i + blockDim.x] = b;
          dst[i + 2 * blockDim.x] = c;
          dst[i + 3 * blockDim.x] = d;
        }
        for (; i < n16; i += blockDim.x) dst[i] = src[i];
      }
      __syncthreads();
    }
    if (threadIdx.x == 0) {
      __threadfence();
      st_release_gpu(gp.flags + gi, gp.epoch);
    }
  }
  // the last copy CTA to finish tells every source owner that its chunk has been read
  __syncthreads();
  if (threadIdx.x == 0 && gp.done_counter) {
    __threadfence();
    const int prev = atomicAdd(gp.done_counter, 1);
    if (prev == gp.n_copy_ctas - 1) {
      for (int c = 0; c < gp.n_chunks; ++c)
        if (gp.peer_done[c]) st_release_sys(gp.peer_done[c], gp.epoch);
    }
  }
}

// Body of a copy CTA in reduce mode: this rank's slice of an fp32 reduce-scatter, read from every
// rank's buffer with plain loads, summed in chunk order and scaled.
__device__ __forceinline__ void reduce_copy_cta(const GatherParams& gp, int cta, volatile int* abort_flag,
                                                int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_ok = 1;
    for (int c = 0; c < gp.n_chunks && s_ok; ++c)
      if (gp.ready && c != gp.first_chunk && !wait_flag(gp.ready + c, gp.epoch, true, abort_flag, status)) s_ok = 0;
  }
  __syncthreads();
  if (s_ok && gp.mc_src != nullptr) {
    // in-switch reduction: one multimem load per 16 bytes brings back the sum over all ranks
    const long n4 = gp.reduce_numel >> 2;
    float4* out = reinterpret_cast<float4*>(gp.reduce_out);
    const float4* src = reinterpret_cast<const float4*>(gp.mc_src);
    const long stride = static_cast<long>(gp.n_copy_ctas) * blockDim.x;
    constexpr int kUnroll = 4;
    for (long base = static_cast<long>(cta) * blockDim.x + threadIdx.x; base < n4; base += stride * kUnroll) {
      float4 v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long i = base + u * stride;
        if (i < n4)
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(v[u].x), "=f"(v[u].y), "=f"(v[u].z), "=f"(v[u].w)
                       : "l"(src + i)
                       : "memory");
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long i = base + u * stride;
        if (i < n4)
          out[i] = make_float4(v[u].x * gp.reduce_scale, v[u].y * gp.reduce_scale, v[u].z * gp.reduce_scale,
                               v[u].w * gp.reduce_scale);
      }
    }
  } else if (s_ok) {
    const long n4 = gp.reduce_numel >> 2;
    float4* out = reinterpret_cast<float4*>(gp.reduce_out);
    const long stride = static_cast<long>(gp.n_copy_ctas) * blockDim.x;
    constexpr int kUnroll = 4;     // elements per thread and pass: kUnroll * ranks 16-byte loads in flight
    for (long base = static_cast<long>(cta) * blockDim.x + threadIdx.x; base < n4; base += stride * kUnroll) {
      float4 v[kUnroll][kMaxPeers];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long i = base + u * stride;
#pragma unroll
        for (int c = 0; c < kMaxPeers; ++c)
          if (c < gp.n_chunks && i < n4) v[u][c] = reinterpret_cast<const float4*>(gp.src[c])[i];
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long i = base + u * stride;
        if (i >= n4) break;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int c = 0; c < kMaxPeers; ++c)
          if (c < gp.n_chunks) {
            acc.x += v[u][c].x;
            acc.y += v[u][c].y;
            acc.z += v[u][c].z;
            acc.w += v[u][c].w;
          }
        acc.x *= gp.reduce_scale;
        acc.y *= gp.reduce_scale;
        acc.z *= gp.reduce_scale;
        acc.w *= gp.reduce_scale;
        out[i] = acc;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && gp.done_counter) {
    __threadfence();
    const int prev = atomicAdd(gp.done_counter, 1);
    if (prev == gp.n_copy_ctas - 1) {
      for (int c = 0; c < gp.n_chunks; ++c)
        if (gp.peer_done[c]) st_release_sys(gp.peer_done[c], gp.epoch);
    }
  }
}

// Work schedule. Items [0, full) are whole tiles. When the last wave would leave most SMs idle,
// its `tail` tiles are each cut into `parts` slices along K (items full .. full + tail * parts):
// every slice leaves its fp32 partial tile in a workspace and bumps a per-tile counter; whichever
// slice arrives last adds the partials in slice order (so the sum does not depend on timing) and
// writes the tile.
struct SplitParams {
  int full = 0;        // number of whole-tile items
  int parts = 1;       // K slices per tail tile
  int kb_per = 0;      // k-blocks per slice
  int items = 0;       // total number of work items
  int prefetch = 0;    // k-blocks of L2 prefetch ahead of the shared-memory loads (0 = off)
  int group_m = 0;     // pair kernel: row tiles that share one column sweep (0 = default)
  int* tile_counter = nullptr;  // pair kernel: zeroed counter that hands out work items (nullptr = static schedule)
  float* workspace = nullptr;   // [tail][parts][4 quarters][BN/32][32 lanes][32] floats
  int* counters = nullptr;      // [tail][4 quarters], zeroed by the launcher
};

struct WorkItem {
  int tile, kb_begin, kb_end, part, tail_index;
};

__device__ __forceinline__ WorkItem decode_item(const SplitParams& kp, int w, int num_kb) {
  WorkItem it;
  if (w < kp.full || kp.parts <= 1) {
    it.tile = w;
    it.kb_begin = 0;
    it.kb_end = num_kb;
    it.part = -1;
    it.tail_index = 0;
  } else {
    const int r = w - kp.full;
    it.tail_index = r / kp.parts;
    it.part = r - it.tail_index * kp.parts;
    it.tile = kp.full + it.tail_index;
    it.kb_begin = it.part * kp.kb_per;
    it.kb_end = min(num_kb, it.kb_begin + kp.kb_per);
  }
  return it;
}

// Epilogue of one warp for one accumulator: TMEM lanes [32 q, 32 q + 32) x BN columns, i.e. rows
// m0 + 32 q .. of the output tile whose first column is n0. `release()` is called (by the whole
// warp) as soon as the accumulator has been read out of TMEM. `part` >= 0 marks a K-slice of a
// split tile; `split_slot` then names its workspace / counter slot. `staging` is the CTA's
// 4 x 4 KB shared-memory staging area.
template <int BN, typename OutT, typename Release>
__device__ __forceinline__ void drain_quarter(uint32_t taddr, uint32_t staging, OutT* __restrict__ D, int M,
                                              int N, int ldd, bool accumulate, bool vec_ok,
                                              bool staged_epilogue, int m0, int n0, int q, int lane,
                                              const ScatterParams& sp, const SplitParams& kp, int part,
                                              int split_slot, Release release) {
  const int row = m0 + q * 32 + lane;
  if (part >= 0) {
    // ---- K-slice of a tail tile: park the fp32 partial, last arriver reduces in slice order
    constexpr int kQuarterFloats = (BN / 32) * 32 * 32;
    float* slot0 = kp.workspace +
                   (static_cast<size_t>(split_slot) * kp.parts * 4 + q) * kQuarterFloats;
    float* mine = slot0 + static_cast<size_t>(part) * 4 * kQuarterFloats;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t v[32];
      tmem_ld_32x32(taddr + c * 32, v);
      tmem_ld_wait();
      float4* dst = reinterpret_cast<float4*>(mine + (c * 32 + lane) * 32);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        dst[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                             __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
    }
    tc_fence_before();
    __threadfence();
    __syncwarp();
    release();
    int prev = 0;
    if (lane == 0) prev = atomicAdd(kp.counters + split_slot * 4 + q, 1);
    prev = __shfl_sync(0xffffffffu, prev, 0);
    if (prev == kp.parts - 1) {
      __threadfence();
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = 0.f;
        for (int pp = 0; pp < kp.parts; ++pp) {
          const float4* src = reinterpret_cast<const float4*>(
              slot0 + static_cast<size_t>(pp) * 4 * kQuarterFloats + (c * 32 + lane) * 32);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 x = __ldcg(src + i);
            f[4 * i] += x.x;
            f[4 * i + 1] += x.y;
            f[4 * i + 2] += x.z;
            f[4 * i + 3] += x.w;
          }
        }
        uint32_t v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(f[j]);
        const int col = n0 + c * 32;
        if (row < M && col < N) {
          OutT* base = D + static_cast<size_t>(row) * ldd;
          store_chunk<OutT>(base + col, v, min(32, N - col), vec_ok, accumulate);
        }
      }
    }
    return;
  }
  if constexpr (sizeof(OutT) == 2) {
    if (sp.n_chunks > 0 || (vec_ok && !accumulate && staged_epilogue)) {
      // The warp's 32 x 64 sub-tile is transposed through shared memory (128B-swizzled,
      // conflict-free both ways) and written 4 rows x 128 B per instruction: whole lines,
      // which is what stores that cross NVLink need (reduce-scatter: the rows' owner
      // receives this partial directly) and what keeps L2 write traffic to full sectors.
      const uint32_t stage_base = staging + q * (32 * 128);
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
          uint32_t v[32];
          tmem_ld_32x32(taddr + c * 64 + hlf * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t chunk = static_cast<uint32_t>(hlf * 4 + j) ^ (lane & 7);
            st_shared_v4(stage_base + lane * 128 + chunk * 16,
                         pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1])),
                         pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3])),
                         pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5])),
                         pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7])));
          }
        }
        __syncwarp();
        const int col = n0 + c * 64 + (lane & 7) * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = i * 4 + (lane >> 3);
          const int grow = m0 + q * 32 + r;
          const uint4 val = ld_shared_v4(stage_base + r * 128 + (((lane & 7) ^ (r & 7)) * 16));
          if (grow < M && col < N) {
            __nv_bfloat16* dst;
            if (sp.n_chunks > 0) {
              const int owner = grow / sp.rows_per_chunk;
              dst = static_cast<__nv_bfloat16*>(sp.dst[owner]) +
                    static_cast<size_t>(grow - owner * sp.rows_per_chunk) * ldd + col;
            } else {
              dst = reinterpret_cast<__nv_bfloat16*>(D) + static_cast<size_t>(grow) * ldd + col;
            }
            *reinterpret_cast<uint4*>(dst) = val;
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      release();
      return;
    }
  }
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t v[32];
    tmem_ld_32x32(taddr + c * 32, v);
    tmem_ld_wait();
    const int col = n0 + c * 32;
    if (row < M && col < N) {
      OutT* base = D + static_cast<size_t>(row) * ldd;
      store_chunk<OutT>(base + col, v, min(32, N - col), vec_ok, accumulate);
    }
  }
  tc_fence_before();
  __syncwarp();
  release();
}

template <int BN, bool A_MN, bool B_MN, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a,
                 const __grid_constant__ CUtensorMap tma_b, OutT* __restrict__ D, int M, int N,
                 int K, int ldd, int accumulate, int* __restrict__ status,
                 const __grid_constant__ GatherParams gp,
                 const __grid_constant__ ScatterParams sp,
                 const __grid_constant__ SplitParams kp,
                 const __grid_constant__ GroupParams gq) {
  using C = Cfg<BN>;
  constexpr int kStages = C::kStages;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];
  __shared__ __align__(8) uint64_t bar_tfull[2];
  __shared__ __align__(8) uint64_t bar_tempty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_m = (M + kBM - 1) / kBM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bar_tfull[s]), 1);
      mbar_init(smem_u32(&bar_tempty[s]), 4);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  pdl_trigger();
  pdl_wait();      // nothing above reads or writes global memory

  // With a fused gather the first `n_copy` CTAs only copy; the rest share the tiles.
  const int m_rot = gp.m_rot + sp.m_rot;
  const int n_items = kp.parts > 1 ? kp.items : (gq.mode == 2 ? num_tiles * gq.n_groups : num_tiles);
  const int n_copy = gp.n_copy_ctas;
  // Grouped launches: work item -> (tile, K range, operand / output offsets); false = nothing to do.
  auto grouped = [&](int w, WorkItem& it, int& tm, int& tn, long& b_rows, long& d_off) -> bool {
    b_rows = 0;
    d_off = 0;
    if (gq.mode == 2) {
      const int e = w / num_tiles;
      it.tile = w - e * num_tiles;
      it.kb_begin = gq.k_begin[e] >> 6;
      it.kb_end = gq.k_end[e] >> 6;
      d_off = static_cast<long>(e) * gq.d_group_elems;
      if (it.kb_end <= it.kb_begin) return false;
    }
    tile_coords(it.tile, tiles_m, tiles_n, tm, tn);
    if (gq.mode == 1) {
      const int g = gq.tile_group[tm];
      if (g < 0) return false;
      b_rows = static_cast<long>(g) * gq.b_group_rows;
    }
    return true;
  };
  const int first_tile = static_cast<int>(blockIdx.x) - n_copy;
  const int tile_step = static_cast<int>(gridDim.x) - n_copy;

  if (first_tile < 0) {
    if (gp.reduce_out) reduce_copy_cta(gp, blockIdx.x, &abort_flag, status);
    else gather_copy_cta(gp, blockIdx.x, &abort_flag, status);
  } else if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int w = first_tile; w < n_items && ok; w += tile_step) {
      WorkItem it = decode_item(kp, w, num_kb);
      int tm, tn;
      long b_rows = 0, d_off = 0;
      if (gq.mode) {
        if (!grouped(w, it, tm, tn, b_rows, d_off)) continue;
      } else {
        tile_coords(it.tile, tiles_m, tiles_n, tm, tn);
      }
      if (m_rot) tm = (tm + m_rot) % tiles_m;
      const int m0 = tm * kBM, n0 = tn * BN;
      const int bq = static_cast<int>(b_rows);
      if (gp.dep == 1) ok = wait_rows(gp, m0, kBM, M, &abort_flag, status);
      if (gp.dep == 2) ok = wait_rows(gp, n0, BN, N, &abort_flag, status);
      if (!ok) break;
      if (gp.dep) fence_proxy_async();  // copied data was written by generic stores; TMA reads it
      for (int kb = it.kb_begin; kb < it.kb_end; ++kb) {
        ok = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1, &abort_flag, status, kTimeoutEmpty);
        if (!ok) break;
        const uint32_t full = smem_u32(&bar_full[stage]);
        const uint32_t sa = smem_base + stage * C::kStageBytes;
        const uint32_t sb = sa + C::kABytes;
        mbar_expect_tx(full, C::kStageBytes);
        const int k0 = kb * kBK;
        if (kp.prefetch > 0 && kb + kp.prefetch < it.kb_end) {
          // warm L2 for a later k-block: the real loads then see L2 latency instead of DRAM's
          const int kf = (kb + kp.prefetch) * kBK;
          if (!A_MN) {
            tma_prefetch_2d(&tma_a, kf, m0);
          } else {
#pragma unroll
            for (int c = 0; c < kBM / 64; ++c) tma_prefetch_2d(&tma_a, m0 + c * 64, kf);
          }
          if (!B_MN) {
            tma_prefetch_2d(&tma_b, kf, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_prefetch_2d(&tma_b, n0 + c * 64, kf);
          }
        }
        if (!A_MN) {
          tma_load_2d(sa, &tma_a, full, k0, m0);
        } else {
#pragma unroll
          for (int c = 0; c < kBM / 64; ++c) tma_load_2d(sa + c * 8192, &tma_a, full, m0 + c * 64, k0);
        }
        if (!B_MN) {
          tma_load_2d(sb, &tma_b, full, k0, n0 + bq);
        } else {
#pragma unroll
          for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * 8192, &tma_b, full, n0 + c * 64, k0 + bq);
        }
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (first_tile >= 0 && warp == 1 && lane == 0) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc_bf16(kBM, BN, A_MN, B_MN);
    int stage = 0;
    uint32_t phase = 0;
    int local = 0;
    bool ok = true;
    for (int w = first_tile; w < n_items && ok; w += tile_step, ++local) {
      WorkItem it = decode_item(kp, w, num_kb);
      if (gq.mode) {
        int tm, tn;
        long b_rows, d_off;
        if (!grouped(w, it, tm, tn, b_rows, d_off)) {
          --local;       // skipped items use no accumulator
          continue;
        }
      }
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ok = mbar_wait(smem_u32(&bar_tempty[acc]), acc_phase ^ 1, &abort_flag, status,
                     kTimeoutTmemEmpty);
      if (!ok) break;
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + acc * BN;
      for (int kb = it.kb_begin; kb < it.kb_end; ++kb) {
        ok = mbar_wait(smem_u32(&bar_full[stage]), phase, &abort_flag, status, kTimeoutFull);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = smem_base + stage * C::kStageBytes;
        const uint32_t sb = sa + C::kABytes;
#pragma unroll
        for (int k = 0; k < kBK / kUK; ++k) {
          // K-major: 16 k = 32 bytes inside the swizzled row; MN-major: 16 k rows = 2048 bytes
          const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, 8192, 1024)
                                   : make_smem_desc(sa + k * 32, 0, 1024);
          const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, 8192, 1024)
                                   : make_smem_desc(sb + k * 32, 0, 1024);
          umma_bf16(tmem_d, da, db, idesc, ((kb - it.kb_begin) | k) != 0);
        }
        umma_commit(smem_u32(&bar_empty[stage]));  // frees the smem stage when the MMAs retire
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) umma_commit(smem_u32(&bar_tfull[acc]));  // accumulator ready for the epilogue
    }
  } else if (first_tile >= 0 && warp >= 4) {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const bool staged_epilogue = (N % 8 == 0);
    const bool vec_ok = (ldd % (16 / (int)sizeof(OutT)) == 0) &&
                        ((reinterpret_cast<uintptr_t>(D) & 15) == 0);
    int local = 0;
    bool ok = true;
    for (int w = first_tile; w < n_items && ok; w += tile_step, ++local) {
      WorkItem it = decode_item(kp, w, num_kb);
      int tm, tn;
      long b_rows = 0, d_off = 0;
      if (gq.mode) {
        if (!grouped(w, it, tm, tn, b_rows, d_off)) {
          --local;
          continue;
        }
      } else {
        tile_coords(it.tile, tiles_m, tiles_n, tm, tn);
      }
      if (m_rot) tm = (tm + m_rot) % tiles_m;
      const int m0 = tm * kBM, n0 = tn * BN;
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ok = mbar_wait(smem_u32(&bar_tfull[acc]), acc_phase, &abort_flag, status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      const uint32_t tempty = smem_u32(&bar_tempty[acc]);
      drain_quarter<BN, OutT>(taddr, smem_base + kStages * C::kStageBytes, D + d_off, M, N, ldd, accumulate != 0, vec_ok,
                              staged_epilogue, m0, n0, q, lane, sp, kp, it.part, it.tail_index, [&]() {
                                if (lane == 0) mbar_arrive(tempty);
                              });
    }
  }

  if (sp.n_chunks > 0 && first_tile >= 0) {
    // ---- reduce-scatter tail: announce, wait for the peers, reduce the own chunk
    __threadfence_system();  // every thread: its tile stores (some to peer memory) are visible
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      const int prev = atomicAdd(sp.cta_counter, 1);
      if (prev == tile_step - 1) {
        for (int p = 0; p < sp.n_chunks; ++p)
          if (p != sp.rank && sp.peer_flag[p]) st_release_sys(sp.peer_flag[p], sp.epoch);
      }
      bool ok = true;
      for (int p = 0; p < sp.n_chunks && ok; ++p)
        if (p != sp.rank) ok = wait_flag(sp.my_flags + p, sp.epoch, true, &abort_flag, status);
      // the own partial is complete once every local CTA has passed the counter
      if (ok) ok = wait_flag(sp.cta_counter, tile_step, false, &abort_flag, status);
    }
    __syncthreads();
    if (!abort_flag) {
      if constexpr (sizeof(OutT) == 2) {
        const long nvec = static_cast<long>(sp.rows_per_chunk) * N / 8;  // N % 8 == 0 is required
        const uint4* own = reinterpret_cast<const uint4*>(sp.dst[sp.rank]);
        uint4* outp = reinterpret_cast<uint4*>(sp.out);
        for (long i = static_cast<long>(first_tile) * kThreads + threadIdx.x; i < nvec;
             i += static_cast<long>(tile_step) * kThreads) {
          float f[8];
          {
            const uint4 raw = own[i];
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 t = __bfloat1622float2(h2[j]);
              f[2 * j] = t.x;
              f[2 * j + 1] = t.y;
            }
          }
          for (int p = 0; p < sp.n_chunks; ++p) {
            if (p == sp.rank) continue;
            const uint4 raw = reinterpret_cast<const uint4*>(sp.recv[p])[i];
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 t = __bfloat1622float2(h2[j]);
              f[2 * j] += t.x;
              f[2 * j + 1] += t.y;
            }
          }
          uint4 o;
          o.x = pack_bf16x2(f[0], f[1]);
          o.y = pack_bf16x2(f[2], f[3]);
          o.z = pack_bf16x2(f[4], f[5]);
          o.w = pack_bf16x2(f[6], f[7]);
          outp[i] = o;
        }
      }
    }
  }

  if (abort_flag) {
    // a wait gave up: let copies that are still in flight land before the CTA's
    // shared memory is handed to someone else
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ------------------------------------------------------------------ CTA-pair kernel
// Same roles as above, but two CTAs of a cluster (one per SM of a TPC) share each 256 x 256
// output tile through `tcgen05.mma.cta_group::2`: each CTA loads its own 128 rows of A and its
// own 128 columns of B (32 KB per k-block instead of 48 KB, which is what the single-CTA kernel
// is bound by) and owns 128 x 256 of the accumulator in its own TMEM. The even CTA issues the
// MMAs for both. Barrier traffic between the two:
//   full[s]    lives in the even CTA; both CTAs' TMA loads count their bytes on it
//   empty[s]   one in each CTA, released together by a commit addressed to both
//   tfull[a]   one in each CTA (both epilogues wait locally), same commit form
//   tempty[a]  lives in the even CTA; the eight epilogue warps of the pair arrive on it
// Work items are handed out dynamically when the launcher provides a counter: the even CTA's
// producer draws the next item number with an atomic add and publishes it through a four-entry
// ring in both CTAs' shared memory (sfull[i] in each CTA, sempty[i] in the even CTA, on which
// the pair's other ten consumers arrive). A cluster that starts late, because its SMs were busy
// with another kernel (a collective running beside the GEMM), then simply takes fewer items
// instead of holding the whole launch back with a fixed share. Without a counter cluster c
// takes items c, c + n_clusters, ... .
struct PairCfg {
  static constexpr int kBN = 256;                       // columns of the pair's tile
  static constexpr int kHalfN = 128;                    // columns of B held by one CTA
  static constexpr int kStages = 6;
  static constexpr int kABytes = kBM * kBK * 2;         // 16 KB
  static constexpr int kBBytes = kHalfN * kBK * 2;      // 16 KB
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingBytes = 4 * 32 * 128;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024;
  static constexpr int kTmemCols = 2 * kBN;
  static constexpr int kGroupM = 8;                     // raster group, in 256-row tiles
  static constexpr int kSched = 4;                      // depth of the work-item ring
  static constexpr int kSchedReaders = 10;              // MMA + 4 epilogue warps here, producer + 4 epilogue warps there
};

__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& tm,
                                                 int& tn) {
  const int per_group = group_m * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * group_m;
  const int gsz = min(group_m, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

template <bool A_MN, bool B_MN, typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tma_a,
                      const __grid_constant__ CUtensorMap tma_b, OutT* __restrict__ D, int M, int N,
                      int K, int ldd, int accumulate, int* __restrict__ status,
                      const __grid_constant__ SplitParams kp, const __grid_constant__ GatherParams gp) {
  using C = PairCfg;
  constexpr int kStages = C::kStages;
  constexpr int BN = C::kBN;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];
  __shared__ __align__(8) uint64_t bar_tfull[2];
  __shared__ __align__(8) uint64_t bar_tempty[2];
  __shared__ __align__(8) uint64_t bar_sfull[PairCfg::kSched];
  __shared__ __align__(8) uint64_t bar_sempty[PairCfg::kSched];
  __shared__ int sched_item[PairCfg::kSched];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();   // 0: issues the MMAs, 1: its partner
  const bool leader = rank == 0;
  // The first n_copy_ctas / 2 clusters of a launch that carries a copy or reduction job (no tile
  // depends on it: gp.dep == 0) only run that job; they take part in the two cluster barriers
  // and in nothing else.
  const int copy_clusters = gp.n_copy_ctas >> 1;
  const bool copy_cluster = static_cast<int>(cluster_id_x()) < copy_clusters;

  const int tiles_m = (M + 2 * kBM - 1) / (2 * kBM);
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);    // the even CTA's producer; bytes from both CTAs
      mbar_init(smem_u32(&bar_empty[s]), 1);   // one commit
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bar_tfull[s]), 1);   // one commit
      mbar_init(smem_u32(&bar_tempty[s]), 8);  // four epilogue warps in each CTA
    }
    for (int s = 0; s < C::kSched; ++s) {
      mbar_init(smem_u32(&bar_sfull[s]), 1);
      mbar_init(smem_u32(&bar_sempty[s]), C::kSchedReaders);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 2 && !copy_cluster) {
    tmem_alloc_pair(smem_u32(&tmem_slot), C::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  // both CTAs' barriers exist before either sends the other a signal
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = copy_cluster ? 0u : tmem_slot;

  const int n_items = kp.parts > 1 ? kp.items : num_tiles;
  const int group_m = kp.group_m > 0 ? kp.group_m : C::kGroupM;
  const int first_tile = static_cast<int>(cluster_id_x()) - copy_clusters;
  const int tile_step = static_cast<int>(num_clusters_x()) - copy_clusters;
  const bool dynamic = kp.tile_counter != nullptr;

  // Next work item of this role (-1: none left, or a wait gave up). `n` counts the items the
  // role has taken so far; every role of the pair sees the same sequence.
  auto next_item = [&](int n) -> int {
    if (!dynamic) {
      const int w = first_tile + n * tile_step;
      return w < n_items ? w : -1;
    }
    const int slot = n % C::kSched;
    const uint32_t sphase = (n / C::kSched) & 1;
    if (!mbar_wait_cluster(smem_u32(&bar_sfull[slot]), sphase, &abort_flag, status, kTimeoutSchedule)) return -1;
    const int w = *reinterpret_cast<volatile int*>(&sched_item[slot]);
    const uint32_t release = mapa_shared(smem_u32(&bar_sempty[slot]), 0);
    if (warp >= 4) {           // epilogue warps come here with all lanes, the other roles with one
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(release);
    } else {
      mbar_arrive_cluster(release);
    }
    return w;
  };
  // The even CTA's producer fills the ring: entry n gets item `w` (already drawn from the counter).
  auto publish_item = [&](int n, int w) -> int {
    const int slot = n % C::kSched;
    const uint32_t sphase = (n / C::kSched) & 1;
    if (!mbar_wait_cluster(smem_u32(&bar_sempty[slot]), sphase ^ 1, &abort_flag, status, kTimeoutSchedule))
      return -1;
    if (w >= n_items) w = -1;
    *reinterpret_cast<volatile int*>(&sched_item[slot]) = w;
    st_shared_cluster_u32(mapa_shared(smem_u32(&sched_item[slot]), 1), static_cast<uint32_t>(w));
    mbar_arrive(smem_u32(&bar_sfull[slot]));
    mbar_arrive_cluster(mapa_shared(smem_u32(&bar_sfull[slot]), 1));
    return w;
  };

  if (copy_cluster) {
    if (gp.reduce_out) reduce_copy_cta(gp, blockIdx.x, &abort_flag, status);
    else gather_copy_cta(gp, blockIdx.x, &abort_flag, status);
  } else if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ producer (one per CTA)
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    // The even CTA's producer draws item n + 1 from the counter before it loads item n and
    // publishes it afterwards: the counter's round trip overlaps the loads.
    const bool scheduler = dynamic && leader;
    int current = scheduler ? publish_item(0, atomicAdd(kp.tile_counter, 1)) : 0;
    for (int n = 0; ok; ++n) {
      const int w = scheduler ? current : next_item(n);
      int drawn = 0;
      if (scheduler && w >= 0) drawn = atomicAdd(kp.tile_counter, 1);
      if (w < 0) break;
      const WorkItem it = decode_item(kp, w, num_kb);
      int tm, tn;
      pair_tile_coords(it.tile, tiles_m, tiles_n, group_m, tm, tn);
      const int m0 = tm * 2 * kBM + static_cast<int>(rank) * kBM;
      const int n0 = tn * BN + static_cast<int>(rank) * C::kHalfN;
      for (int kb = it.kb_begin; kb < it.kb_end; ++kb) {
        ok = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1, &abort_flag, status, kTimeoutEmpty);
        if (!ok) break;
        const uint32_t full_local = smem_u32(&bar_full[stage]);
        const uint32_t full = mapa_shared(full_local, 0);
        const uint32_t sa = smem_base + stage * C::kStageBytes;
        const uint32_t sb = sa + C::kABytes;
        if (leader) mbar_expect_tx(full_local, 2 * C::kStageBytes);
        const int k0 = kb * kBK;
        if (!A_MN) {
          tma_load_2d_pair(sa, &tma_a, full, k0, m0);
        } else {
#pragma unroll
          for (int c = 0; c < kBM / 64; ++c) tma_load_2d_pair(sa + c * 8192, &tma_a, full, m0 + c * 64, k0);
        }
        if (!B_MN) {
          tma_load_2d_pair(sb, &tma_b, full, k0, n0);
        } else {
#pragma unroll
          for (int c = 0; c < C::kHalfN / 64; ++c)
            tma_load_2d_pair(sb + c * 8192, &tma_b, full, n0 + c * 64, k0);
        }
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (scheduler && ok) current = publish_item(n + 1, drawn);
    }
    // The stage releases come from the even CTA's commits: wait until every one addressed to
    // this CTA has landed, so that none arrives after the CTA has left.
    for (int s = 0; s < kStages && ok; ++s) {
      ok = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1, &abort_flag, status, kTimeoutEmpty);
      if (++stage == kStages) {
        stage = 0;
        phase ^= 1;
      }
    }
  } else if (leader && warp == 1 && lane == 0) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    constexpr uint32_t idesc = make_idesc_bf16(2 * kBM, BN, A_MN, B_MN);
    int stage = 0;
    uint32_t phase = 0;
    int local = 0;
    bool ok = true;
    for (; ok; ++local) {
      const int w = next_item(local);
      if (w < 0) break;
      const WorkItem it = decode_item(kp, w, num_kb);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ok = mbar_wait_cluster(smem_u32(&bar_tempty[acc]), acc_phase ^ 1, &abort_flag, status,
                             kTimeoutTmemEmpty);
      if (!ok) break;
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + acc * BN;
      for (int kb = it.kb_begin; kb < it.kb_end; ++kb) {
        ok = mbar_wait_cluster(smem_u32(&bar_full[stage]), phase, &abort_flag, status, kTimeoutFull);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = smem_base + stage * C::kStageBytes;
        const uint32_t sb = sa + C::kABytes;
#pragma unroll
        for (int k = 0; k < kBK / kUK; ++k) {
          const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, 8192, 1024)
                                   : make_smem_desc(sa + k * 32, 0, 1024);
          const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, 8192, 1024)
                                   : make_smem_desc(sb + k * 32, 0, 1024);
          umma_bf16_pair(tmem_d, da, db, idesc, ((kb - it.kb_begin) | k) != 0);
        }
        umma_commit_pair(smem_u32(&bar_empty[stage]), 3);  // frees the stage in both CTAs
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) umma_commit_pair(smem_u32(&bar_tfull[acc]), 3);  // both epilogues may read
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    const bool staged_epilogue = (N % 8 == 0);
    const bool vec_ok = (ldd % (16 / (int)sizeof(OutT)) == 0) &&
                        ((reinterpret_cast<uintptr_t>(D) & 15) == 0);
    const ScatterParams no_scatter;
    int local = 0;
    bool ok = true;
    for (; ok; ++local) {
      const int w = next_item(local);
      if (w < 0) break;
      const WorkItem it = decode_item(kp, w, num_kb);
      int tm, tn;
      pair_tile_coords(it.tile, tiles_m, tiles_n, group_m, tm, tn);
      const int m0 = tm * 2 * kBM + static_cast<int>(rank) * kBM;
      const int n0 = tn * BN;
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ok = mbar_wait_cluster(smem_u32(&bar_tfull[acc]), acc_phase, &abort_flag, status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      const uint32_t tempty = mapa_shared(smem_u32(&bar_tempty[acc]), 0);
      drain_quarter<BN, OutT>(taddr, smem_base + kStages * C::kStageBytes, D, M, N, ldd, accumulate != 0, vec_ok,
                              staged_epilogue, m0, n0, q, lane, no_scatter, kp, it.part,
                              it.tail_index * 2 + static_cast<int>(rank), [&]() {
                                if (lane == 0) mbar_arrive_cluster(tempty);
                              });
    }
  }

  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  // neither CTA leaves (or frees tensor memory) while its partner may still signal its
  // barriers or read its shared memory
  cluster_sync_all();
  if (warp == 2 && !copy_cluster) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, C::kTmemCols);
  }
}

// ------------------------------------------------------------------ skinny GEMM: K split over a cluster
// Decode-time projections have at most 128 rows and a handful of 64-column tiles, so a launch of
// one CTA per tile leaves most SMs idle while each busy one streams its whole K range through a
// single TMA queue. Here a cluster of S CTAs (2..8) shares one 128 x 64 tile: CTA r accumulates
// k-blocks [r * per, (r + 1) * per) in its own tensor memory, the CTAs with r > 0 then write
// their fp32 partial into CTA 0's shared memory (distributed shared memory stores), the cluster
// meets at a barrier and CTA 0 adds the S partials in rank order and writes the tile. No global
// workspace, counters or second kernel. A, B K-major.
struct KSplitCfg {
  static constexpr int kBN = 64;
  static constexpr int kStages = 4;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = kBN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;              // 24 KB
  static constexpr int kMaxSplit = 8;
  static constexpr int kQuarterBytes = 32 * kBN * 4;                 // 32 rows of one CTA's fp32 tile: 8 KB
  static constexpr int kPartialArea = 12 * kQuarterBytes;            // room for the partials of ranks 1..S-1
  static constexpr int kSmemBytes = kStages * kStageBytes + kPartialArea + 1024;
  static constexpr int kTmemCols = 64;
};

// Byte offset inside a partial (only the row quarters below M are stored) of the 16-byte piece `i` (0..7) of lane `lane`'s 32-float
// chunk `c` of lane quarter `q`; pieces are XOR-swizzled so that neither the remote writer nor
// the local reader has bank conflicts.
__device__ __forceinline__ uint32_t partial_offset(int q, int c, int lane, int i) {
  return static_cast<uint32_t>(((q * (KSplitCfg::kBN / 32) + c) * 32 + lane) * 128 + ((i ^ (lane & 7)) << 4));
}

template <typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_ksplit_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                        OutT* __restrict__ D, int M, int N, int K, int ldd, int accumulate, int split,
                        int* __restrict__ status) {
  using C = KSplitCfg;
  constexpr int kStages = C::kStages;
  constexpr int BN = C::kBN;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];
  __shared__ __align__(8) uint64_t bar_tfull;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t partial_base = smem_base + kStages * C::kStageBytes;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());
  const int tile = static_cast<int>(cluster_id_x());

  const int tiles_n = (N + BN - 1) / BN;
  const int tm = tile / tiles_n, tn = tile - tm * tiles_n;
  const int m0 = tm * kBM, n0 = tn * BN;
  const int num_kb = (K + kBK - 1) / kBK;
  const int per = (num_kb + split - 1) / split;
  const int kb_begin = rank * per;
  const int kb_end = min(num_kb, kb_begin + per);
  const bool has_work = kb_end > kb_begin;
  const int quarters = (min(M - m0, kBM) + 31) / 32;                 // row quarters that hold rows of D
  const uint32_t partial_bytes = static_cast<uint32_t>(quarters) * C::kQuarterBytes;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_tfull), 1);
    fence_barrier_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  pdl_trigger();
  pdl_wait();      // nothing above reads or writes global memory

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    for (int kb = kb_begin; kb < kb_end; ++kb) {
      if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1, &abort_flag, status, kTimeoutEmpty)) break;
      const uint32_t full = smem_u32(&bar_full[stage]);
      const uint32_t sa = smem_base + stage * C::kStageBytes;
      mbar_expect_tx(full, C::kStageBytes);
      tma_load_2d(sa, &tma_a, full, kb * kBK, m0);
      tma_load_2d(sa + C::kABytes, &tma_b, full, kb * kBK, n0);
      if (++stage == kStages) {
        stage = 0;
        phase ^= 1;
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc_bf16(kBM, BN, false, false);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int kb = kb_begin; kb < kb_end && ok; ++kb) {
      ok = mbar_wait(smem_u32(&bar_full[stage]), phase, &abort_flag, status, kTimeoutFull);
      if (!ok) break;
      tc_fence_after();
      const uint32_t sa = smem_base + stage * C::kStageBytes;
      const uint32_t sb = sa + C::kABytes;
#pragma unroll
      for (int k = 0; k < kBK / kUK; ++k)
        umma_bf16(tmem_base, make_smem_desc(sa + k * 32, 0, 1024), make_smem_desc(sb + k * 32, 0, 1024), idesc,
                  ((kb - kb_begin) | k) != 0);
      umma_commit(smem_u32(&bar_empty[stage]));
      if (++stage == kStages) {
        stage = 0;
        phase ^= 1;
      }
    }
    if (ok && has_work) umma_commit(smem_u32(&bar_tfull));
  } else if (warp >= 4 && rank != 0 && has_work) {
    // ------------------------------------------------------------ partial -> CTA 0's shared memory
    const int q = warp & 3;
    bool ok = mbar_wait(smem_u32(&bar_tfull), 0, &abort_flag, status, kTimeoutTmemFull);
    ok = __all_sync(0xffffffffu, ok);
    if (ok && m0 + q * 32 < M) {     // row quarters past M hold zeros nobody reads
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
      const uint32_t dst = mapa_shared(partial_base + (rank - 1) * partial_bytes, 0);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 8; ++i)
          st_shared_cluster_v4(dst + partial_offset(q, c, lane, i), v[4 * i], v[4 * i + 1], v[4 * i + 2],
                               v[4 * i + 3]);
      }
    }
    tc_fence_before();
  }

  // every partial is in place (or its CTA gave up) before CTA 0 reads them
  cluster_sync_all();

  if (warp >= 4 && rank == 0 && !abort_flag) {
    // ------------------------------------------------------------ CTA 0: sum in rank order, write the tile
    const int q = warp & 3;
    const bool vec_ok = (ldd % (16 / (int)sizeof(OutT)) == 0) && ((reinterpret_cast<uintptr_t>(D) & 15) == 0);
    bool ok = mbar_wait(smem_u32(&bar_tfull), 0, &abort_flag, status, kTimeoutTmemFull);
    ok = __all_sync(0xffffffffu, ok);
    const int row = m0 + q * 32 + lane;
    if (ok && m0 + q * 32 < M) {
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + c * 32, v);
        tmem_ld_wait();
        for (int p = 1; p < split; ++p) {
          if (p * per >= num_kb) break;      // that rank had no k-blocks
          const uint32_t src = partial_base + (p - 1) * partial_bytes;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint4 x = ld_shared_v4(src + partial_offset(q, c, lane, i));
            v[4 * i] = __float_as_uint(__uint_as_float(v[4 * i]) + __uint_as_float(x.x));
            v[4 * i + 1] = __float_as_uint(__uint_as_float(v[4 * i + 1]) + __uint_as_float(x.y));
            v[4 * i + 2] = __float_as_uint(__uint_as_float(v[4 * i + 2]) + __uint_as_float(x.z));
            v[4 * i + 3] = __float_as_uint(__uint_as_float(v[4 * i + 3]) + __uint_as_float(x.w));
          }
        }
        const int col = n0 + c * 32;
        if (row < M && col < N)
          store_chunk<OutT>(D + static_cast<size_t>(row) * ldd + col, v, min(32, N - col), vec_ok,
                            accumulate != 0);
      }
    }
    tc_fence_before();
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

// ------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Programmatic dependent launch of the plain single-CTA and split-K launches (HB_GEMM_PDL=0: off).
bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* env = getenv("HB_GEMM_PDL");
    on = (env && env[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

constexpr int kDefaultL2Prefetch = 0;
// k-blocks of L2 prefetch issued ahead of the pipeline (HB_GEMM_L2_PREFETCH overrides; 0 = off).
int l2_prefetch_distance() {
  static int dist = -1;
  if (dist < 0) {
    const char* env = getenv("HB_GEMM_L2_PREFETCH");
    dist = env ? atoi(env) : kDefaultL2Prefetch;
    if (dist < 0 || dist > 64) dist = 0;
  }
  return dist;
}

// Scratch for the split-K tail (partials + arrival counters), one fixed-size slot per
// (device, stream) so GEMMs on different streams never share it. A slot is allocated the first
// time a stream needs one, outside of stream capture; while a stream is being captured into a
// CUDA graph it uses a slot set aside for graphs (see below).
constexpr size_t kSplitWsBytes = size_t(20) << 20;   // >= 148 slices x 128 x 256 fp32
constexpr int kSplitCounters = 1024;
// pseudo stream handle that names the per-device slot used by captured graphs
static const cudaStream_t kGraphSlot = reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(0x1));

cudaError_t split_workspace(size_t bytes, int n_counters, cudaStream_t stream, float** ws, int** counters) {
  struct Slot {
    int dev;
    cudaStream_t stream;
    float* ws;
    int* counters;
  };
  static std::vector<Slot> slots;
  static std::mutex lock;
  if (bytes > kSplitWsBytes || n_counters > kSplitCounters) return cudaErrorInvalidValue;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> hold(lock);
  for (const Slot& s : slots) {
    if (s.dev == dev && s.stream == stream) {
      *ws = s.ws;
      *counters = s.counters;
      return cudaSuccess;
    }
  }
  // A stream that is being captured cannot allocate. It uses the device's graph slot, which is
  // created together with the first ordinary slot (so: run one GEMM eagerly before capturing).
  // All captured graphs of a device share that slot: replay them on one stream at a time.
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    (void)cudaGetLastError();
    for (const Slot& s : slots) {
      if (s.dev == dev && s.stream == kGraphSlot) {
        *ws = s.ws;
        *counters = s.counters;
        return cudaSuccess;
      }
    }
    return cudaErrorStreamCaptureUnsupported;
  }
  if (slots.size() >= 32) return cudaErrorMemoryAllocation;   // bounded: 32 x 20 MB
  bool have_graph_slot = false;
  for (const Slot& s : slots) have_graph_slot |= (s.dev == dev && s.stream == kGraphSlot);
  if (!have_graph_slot) {
    Slot gs{dev, kGraphSlot, nullptr, nullptr};
    if (cudaMalloc(&gs.ws, kSplitWsBytes) == cudaSuccess) {
      if (cudaMalloc(&gs.counters, sizeof(int) * kSplitCounters) == cudaSuccess) {
        slots.push_back(gs);
      } else {
        cudaFree(gs.ws);
      }
    }
    (void)cudaGetLastError();
  }
  Slot s{dev, stream, nullptr, nullptr};
  e = cudaMalloc(&s.ws, kSplitWsBytes);
  if (e != cudaSuccess) return e;
  e = cudaMalloc(&s.counters, sizeof(int) * kSplitCounters);
  if (e != cudaSuccess) {
    cudaFree(s.ws);
    return e;
  }
  slots.push_back(s);
  *ws = s.ws;
  *counters = s.counters;
  return cudaSuccess;
}

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess) return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

}  // namespace

// 2-D bf16 tensor map over a row-major [rows, cols] array with leading dimension `ld`
// (elements), box = [box_rows, box_cols], 128-byte swizzle, zero fill out of range.
bool make_tmap_bf16_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                       uint64_t ld, uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  // The encode call is a driver-API entry point: it needs the primary context current in the
  // calling thread. Threads that have not issued a runtime call yet (autograd's backward
  // workers) get it bound here, once.
  thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return false;
    (void)cudaFree(nullptr);
    ctx_bound = true;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "halite_b200: cuTensorMapEncodeTiled failed (%d): rows=%llu cols=%llu ld=%llu box=%ux%u base=%p\n",
            (int)r, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld,
            box_rows, box_cols, base);
  return r == CUDA_SUCCESS;
}

namespace {

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

// SMs that launches whose CTAs spin on another GPU's progress (the tile-dependent gather mode and the
// scatter mode) leave free. Such a kernel holds every SM it runs on until its peer catches up; when the
// peer is itself held back by a collective of ANOTHER process group whose kernel cannot become resident
// on some GPU because a spinning kernel fills it, the ranks wait in a circle. With a margin at least as
// large as the collective library's CTA count, those kernels always find an SM.
int g_peer_wait_sm_margin = 0;

int peer_wait_sm_count() {
  const int n = sm_count() - g_peer_wait_sm_margin;
  return n < 8 ? 8 : n;
}

template <int BN, bool A_MN, bool B_MN, typename OutT>
cudaError_t launch(const GemmArgs& g) {
  using C = Cfg<BN>;
  CUtensorMap ta, tb;
  bool ok;
  if (!A_MN) ok = make_tmap_bf16_2d(&ta, g.a, g.M, g.K, g.lda, kBM, kBK);
  else       ok = make_tmap_bf16_2d(&ta, g.a, g.K, g.M, g.lda, kBK, 64);
  if (!ok) return cudaErrorInvalidPitchValue;
  GroupParams gq;
  if (g.group) {
    gq = *g.group;
    if (g.gather || g.scatter) return cudaErrorInvalidValue;
    if (gq.mode == 1) {
      // a K-major B is addressed by (k, n + group * N): rows past N would belong to the next expert, which is
      // harmless (masked columns); an MN-major B is addressed by (n, k + group * K), so K must fill whole k-blocks
      if (!gq.tile_group || gq.b_group_rows <= 0 || gq.b_total_rows <= 0 || (B_MN && g.K % kBK)) return cudaErrorInvalidValue;
    } else if (gq.mode == 2) {
      if (!A_MN || !B_MN || !gq.k_begin || !gq.k_end || gq.n_groups <= 0 || gq.d_group_elems % 8)
        return cudaErrorInvalidValue;
    } else {
      return cudaErrorInvalidValue;
    }
  }
  const uint64_t b_rows = (gq.mode == 1) ? static_cast<uint64_t>(gq.b_total_rows)
                                         : static_cast<uint64_t>(B_MN ? g.K : g.N);
  if (!B_MN) ok = make_tmap_bf16_2d(&tb, g.b, b_rows, g.K, g.ldb, BN, kBK);
  else       ok = make_tmap_bf16_2d(&tb, g.b, b_rows, g.N, g.ldb, kBK, 64);
  if (!ok) return cudaErrorInvalidPitchValue;

  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, OutT>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::kSmemBytes);
    if (e != cudaSuccess) {
      fprintf(stderr, "halite_b200: cudaFuncSetAttribute failed: %s\n", cudaGetErrorString(e));
      return e;
    }
    attr_set = true;
  }
  (void)cudaGetLastError();  // do not report an error left behind by an earlier, unrelated call
  int tiles = ((g.M + kBM - 1) / kBM) * ((g.N + BN - 1) / BN);
  if (gq.mode == 2) tiles *= gq.n_groups;
  GatherParams gp;
  if (g.gather) gp = *g.gather;
  int grid;
  if (gp.n_copy_ctas > 0) {
    // every CTA must be resident at once (compute CTAs wait on copy CTAs): one CTA per SM
    if (gp.n_copy_ctas >= sm_count() || gp.granule_bytes % 16 || gp.chunk_bytes % 16)
      return cudaErrorInvalidValue;
    if (gp.reduce_out && (gp.reduce_numel % 4 || (reinterpret_cast<uintptr_t>(gp.reduce_out) & 15)))
      return cudaErrorInvalidValue;
    const int sms = gp.dep != 0 ? peer_wait_sm_count() : sm_count();
    if (gp.n_copy_ctas >= sms) return cudaErrorInvalidValue;
    const int compute = tiles < sms - gp.n_copy_ctas ? tiles : sms - gp.n_copy_ctas;
    grid = compute + gp.n_copy_ctas;
    if (gp.done_counter) cudaMemsetAsync(gp.done_counter, 0, sizeof(int), g.stream);
  } else {
    const int sms = g.scatter ? peer_wait_sm_count() : sm_count();
    grid = tiles < sms ? tiles : sms;
    if (g.max_ctas > 0 && grid > g.max_ctas) grid = g.max_ctas;
  }
  SplitParams kp;
  kp.prefetch = l2_prefetch_distance();
  if (!g.gather && !g.scatter && !g.group) {
    // cut the tiles of a mostly idle last wave along K (see SplitParams)
    const int base = (g.max_ctas > 0 && g.max_ctas < sm_count()) ? g.max_ctas : sm_count();
    const int num_kb = (g.K + kBK - 1) / kBK;
    const int rem = tiles % base;
    // only for the tail of a multi-wave launch: slicing a launch that does not even fill the
    // GPU once costs more (fixed per-CTA set-up, partials through memory) than it recovers
    if (tiles > base && rem > 0 && rem * 2 <= base && num_kb >= 16) {
      int parts = base / rem;
      if (parts > 8) parts = 8;
      while (parts > 1 && ((num_kb + parts - 1) / parts < 8 ||
                           (parts - 1) * ((num_kb + parts - 1) / parts) >= num_kb))
        --parts;   // every slice gets at least 8 k-blocks and none is empty
      if (parts > 1) {
        const size_t ws_bytes = static_cast<size_t>(rem) * parts * kBM * BN * sizeof(float);
        float* ws = nullptr;
        int* counters = nullptr;
        if (split_workspace(ws_bytes, rem * 4, g.stream, &ws, &counters) == cudaSuccess) {
          kp.full = tiles - rem;
          kp.parts = parts;
          kp.kb_per = (num_kb + parts - 1) / parts;
          kp.items = kp.full + rem * parts;
          kp.workspace = ws;
          kp.counters = counters;
          cudaMemsetAsync(counters, 0, sizeof(int) * rem * 4, g.stream);
          grid = kp.items < base ? kp.items : base;
        }
      }
    }
  }
  ScatterParams sp;
  if (g.scatter) {
    sp = *g.scatter;
    if (sizeof(OutT) != 2 || sp.n_chunks > kMaxPeers || g.N % 8 || g.ldd != g.N ||
        sp.rows_per_chunk * sp.n_chunks != g.M || !sp.cta_counter)
      return cudaErrorInvalidValue;
    cudaMemsetAsync(sp.cta_counter, 0, sizeof(int), g.stream);
  }
  if (!g.gather && !g.scatter && !g.group && kp.parts <= 1 && pdl_enabled()) {
    // plain launch with nothing enqueued in front of it (no counter memset): let it start under
    // the previous kernel's tail
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = g.stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, ta, tb, static_cast<OutT*>(g.d), g.M, g.N, g.K, g.ldd,
                              g.accumulate ? 1 : 0, g.status, gp, sp, kp, gq);
  }
  kern<<<grid, kThreads, C::kSmemBytes, g.stream>>>(ta, tb, static_cast<OutT*>(g.d), g.M, g.N, g.K,
                                                    g.ldd, g.accumulate ? 1 : 0, g.status, gp, sp, kp, gq);
  return cudaGetLastError();
}

template <int BN, typename OutT>
cudaError_t dispatch_layout(const GemmArgs& g) {
  if (!g.a_mn_major && !g.b_mn_major) return launch<BN, false, false, OutT>(g);
  if (!g.a_mn_major && g.b_mn_major) return launch<BN, false, true, OutT>(g);
  if (g.a_mn_major && g.b_mn_major) return launch<BN, true, true, OutT>(g);
  return launch<BN, true, false, OutT>(g);
}

// Dynamic hand-out of work items in the pair kernel; HB_GEMM_DYNAMIC=0 keeps the fixed shares.
// Fixed shares keep neighbouring clusters on neighbouring tiles (best L2 reuse) and are the
// default; the counter-driven hand-out pays off when another kernel (a collective) holds some
// SMs while the GEMM runs, and is switched on by the data-parallel wrapper. HB_GEMM_DYNAMIC=0/1
// overrides both.
int g_dynamic_schedule = -1;   // -1: not decided yet, 0 / 1: off / on
bool g_dynamic_forced = false;

bool dynamic_schedule_enabled() {
  if (g_dynamic_schedule < 0) {
    const char* env = getenv("HB_GEMM_DYNAMIC");
    g_dynamic_forced = env != nullptr;
    g_dynamic_schedule = (env && env[0] == '1') ? 1 : 0;
  }
  return g_dynamic_schedule == 1;
}

int max_pair_clusters(const void* kern, int smem_bytes) {
  // how many 2-CTA clusters of this kernel the device can hold at once
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sm_count(), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
    (void)cudaGetLastError();
    n = sm_count() / 2;
  }
  return n < sm_count() / 2 ? n : sm_count() / 2;
}

template <bool A_MN, bool B_MN, typename OutT>
cudaError_t launch_pair(const GemmArgs& g) {
  using C = PairCfg;
  CUtensorMap ta, tb;
  bool ok;
  if (!A_MN) ok = make_tmap_bf16_2d(&ta, g.a, g.M, g.K, g.lda, kBM, kBK);
  else       ok = make_tmap_bf16_2d(&ta, g.a, g.K, g.M, g.lda, kBK, 64);
  if (!ok) return cudaErrorInvalidPitchValue;
  if (!B_MN) ok = make_tmap_bf16_2d(&tb, g.b, g.N, g.K, g.ldb, C::kHalfN, kBK);
  else       ok = make_tmap_bf16_2d(&tb, g.b, g.K, g.N, g.ldb, kBK, 64);
  if (!ok) return cudaErrorInvalidPitchValue;

  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN, OutT>;
  static int clusters_max = 0;
  if (clusters_max == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) {
      fprintf(stderr, "halite_b200: cudaFuncSetAttribute (pair kernel) failed: %s\n", cudaGetErrorString(e));
      return e;
    }
    clusters_max = max_pair_clusters(reinterpret_cast<const void*>(kern), C::kSmemBytes);
  }
  (void)cudaGetLastError();
  const int tiles = ((g.M + 2 * kBM - 1) / (2 * kBM)) * ((g.N + C::kBN - 1) / C::kBN);
  GatherParams gp;
  if (g.gather) {
    gp = *g.gather;
    // only jobs no tile waits for, on whole clusters, leaving at least half of the machine to the tiles
    if (gp.dep != 0 || gp.n_copy_ctas % 2 || gp.n_copy_ctas / 2 * 2 > clusters_max) return cudaErrorInvalidValue;
    if (gp.reduce_out && (gp.reduce_numel % 4 || (reinterpret_cast<uintptr_t>(gp.reduce_out) & 15)))
      return cudaErrorInvalidValue;
    if (gp.done_counter) cudaMemsetAsync(gp.done_counter, 0, sizeof(int), g.stream);
  }
  const int copy_clusters = gp.n_copy_ctas / 2;
  const int compute_max = clusters_max - copy_clusters;
  int clusters = tiles < compute_max ? tiles : compute_max;
  SplitParams kp;
  // counters[0] hands out work items; the rest are the split tiles' arrival counters
  float* ws = nullptr;
  int* counters = nullptr;
  const bool have_ws = split_workspace(0, 1, g.stream, &ws, &counters) == cudaSuccess;
  int n_counters = 0;
  if (have_ws && dynamic_schedule_enabled() && tiles > compute_max) {
    kp.tile_counter = counters;
    n_counters = 1;
  }
  if (have_ws) {
    // same tail treatment as the single-CTA kernel, counted in clusters
    const int base = compute_max;
    const int num_kb = (g.K + kBK - 1) / kBK;
    const int rem = tiles % base;
    if (tiles > base && rem > 0 && rem * 2 <= base && num_kb >= 16) {
      int parts = base / rem;
      if (parts > 8) parts = 8;
      while (parts > 1 && ((num_kb + parts - 1) / parts < 8 ||
                           (parts - 1) * ((num_kb + parts - 1) / parts) >= num_kb))
        --parts;
      const size_t ws_bytes = static_cast<size_t>(rem) * parts * 2 * kBM * C::kBN * sizeof(float);
      if (parts > 1 && ws_bytes <= kSplitWsBytes && 1 + rem * 8 <= kSplitCounters) {
        kp.full = tiles - rem;
        kp.parts = parts;
        kp.kb_per = (num_kb + parts - 1) / parts;
        kp.items = kp.full + rem * parts;
        kp.workspace = ws;
        kp.counters = counters + 1;
        n_counters = 1 + rem * 8;
        clusters = kp.items < base ? kp.items : base;
      }
    }
  }
  if (n_counters > 0) cudaMemsetAsync(counters, 0, sizeof(int) * n_counters, g.stream);
  kern<<<2 * (clusters + copy_clusters), kThreads, C::kSmemBytes, g.stream>>>(
      ta, tb, static_cast<OutT*>(g.d), g.M, g.N, g.K, g.ldd, g.accumulate ? 1 : 0, g.status, kp, gp);
  return cudaGetLastError();
}

template <typename OutT>
cudaError_t dispatch_pair(const GemmArgs& g) {
  if (!g.a_mn_major && !g.b_mn_major) return launch_pair<false, false, OutT>(g);
  if (!g.a_mn_major && g.b_mn_major) return launch_pair<false, true, OutT>(g);
  if (g.a_mn_major && g.b_mn_major) return launch_pair<true, true, OutT>(g);
  return launch_pair<true, false, OutT>(g);
}

template <typename OutT>
cudaError_t launch_ksplit(const GemmArgs& g, int split) {
  using C = KSplitCfg;
  CUtensorMap ta, tb;
  if (!make_tmap_bf16_2d(&ta, g.a, g.M, g.K, g.lda, kBM, kBK)) return cudaErrorInvalidPitchValue;
  if (!make_tmap_bf16_2d(&tb, g.b, g.N, g.K, g.ldb, C::kBN, kBK)) return cudaErrorInvalidPitchValue;
  auto kern = gemm_bf16_ksplit_kernel<OutT>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  (void)cudaGetLastError();
  const int tiles = ((g.M + kBM - 1) / kBM) * ((g.N + C::kBN - 1) / C::kBN);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * split, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = g.stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = split;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, ta, tb, static_cast<OutT*>(g.d), g.M, g.N, g.K, g.ldd,
                            g.accumulate ? 1 : 0, split, g.status);
}

// How many clusters of `size` CTAs of the split kernel the device holds at once (clusters are
// placed on whole TPCs inside one GPC, so this is less than SMs / size for most sizes).
int ksplit_max_clusters(int size) {
  static int cached[KSplitCfg::kMaxSplit + 1] = {};
  if (cached[size] == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count() / size * size, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = KSplitCfg::kSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = size;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    auto kern = gemm_bf16_ksplit_kernel<__nv_bfloat16>;
    int n = 0;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, KSplitCfg::kSmemBytes) !=
            cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, reinterpret_cast<const void*>(kern), &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = sm_count() / size / 2;   // conservative guess
    }
    cached[size] = n;
  }
  return cached[size];
}

// K split for skinny K-major problems: the largest power-of-two cluster whose clusters are all
// resident at once (one wave), as long as every CTA keeps at least four k-blocks and the partials
// fit CTA 0's shared memory. Odd sizes waste the second SM of a TPC and measured slower.
int ksplit_factor(const GemmArgs& g) {
  if (g.a_mn_major || g.b_mn_major || g.M > kBM) return 1;
  const int tiles = (g.N + KSplitCfg::kBN - 1) / KSplitCfg::kBN;
  const int num_kb = (g.K + kBK - 1) / kBK;
  const int quarters = (g.M + 31) / 32;
  const int fit = 1 + KSplitCfg::kPartialArea / (quarters * KSplitCfg::kQuarterBytes);
  for (int split = KSplitCfg::kMaxSplit; split >= 2; split /= 2) {
    if (split > fit || split > num_kb / 4) continue;
    if ((split - 1) * ((num_kb + split - 1) / split) >= num_kb) continue;   // a rank without k-blocks
    if (tiles <= ksplit_max_clusters(split)) return split;
  }
  return 1;
}

// The pair kernel is chosen for plain GEMMs that give every SM pair at least one 256 x 256 tile.
// HB_GEMM_PAIR=0 turns it off.
bool pair_kernel_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* env = getenv("HB_GEMM_PAIR");
    on = (env && env[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

}  // namespace

namespace {

struct FlagPtrs {
  int* p[kMaxPeers * 2];
};

__global__ void signal_flags_kernel(FlagPtrs ptrs, int n, int epoch) {
  if (threadIdx.x < n && ptrs.p[threadIdx.x]) {
    __threadfence_system();
    st_release_sys(ptrs.p[threadIdx.x], epoch);
  }
}

__global__ void wait_flags_kernel(const int* flags, int n, int epoch, int* status) {
  __shared__ int abort_flag;
  if (threadIdx.x == 0) abort_flag = 0;
  __syncthreads();
  if (threadIdx.x < n) wait_flag(flags + threadIdx.x, epoch, true, &abort_flag, status);
}

}  // namespace

// Write `epoch` (system scope, after a system fence) to up to 16 flag words, which may live in
// peer memory. Stream-ordered: everything enqueued before it on `stream` is visible first.
cudaError_t signal_flags(const int64_t* ptrs, int n, int epoch, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  if (n > kMaxPeers * 2) return cudaErrorInvalidValue;
  FlagPtrs fp = {};
  for (int i = 0; i < n; ++i) fp.p[i] = reinterpret_cast<int*>(ptrs[i]);
  signal_flags_kernel<<<1, 32, 0, stream>>>(fp, n, epoch);
  return cudaGetLastError();
}

// Block the stream until flags[0..n) >= epoch (bounded: records kTimeoutPeerFlag in *status
// and returns after the wait budget instead of spinning forever).
cudaError_t wait_flags(const int* flags, int n, int epoch, int* status, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  if (n > 32) return cudaErrorInvalidValue;
  wait_flags_kernel<<<1, 32, 0, stream>>>(flags, n, epoch, status);
  return cudaGetLastError();
}

void gemm_set_peer_wait_sm_margin(int sms) {
  g_peer_wait_sm_margin = sms < 0 ? 0 : (sms > sm_count() / 2 ? sm_count() / 2 : sms);
}

int gemm_peer_wait_sm_margin() { return g_peer_wait_sm_margin; }

void gemm_set_dynamic_schedule(bool on, bool force) {
  (void)dynamic_schedule_enabled();   // reads the environment once
  if (g_dynamic_forced && !force) return;
  g_dynamic_schedule = on ? 1 : 0;
}

int gemm_pick_bn(int M, int N) {
  if (N <= 64) return 64;
  const int tm = (M + kBM - 1) / kBM;
  const int t256 = tm * ((N + 255) / 256);
  // prefer the wide tile once it still fills the machine
  if (t256 >= sm_count()) return 256;
  // skinny problems (decode: one row of tiles) are bound by how many SMs pull weights at once:
  // narrower tiles put more CTAs on the job
  const int t128 = tm * ((N + 127) / 128);
  if (N > 128 && 2 * t128 > sm_count()) return 128;
  return 64;
}

cudaError_t gemm_bf16(const GemmArgs& g) {
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return cudaSuccess;
  // TMA needs 16-byte aligned bases and row strides
  if ((reinterpret_cast<uintptr_t>(g.a) & 15) || (reinterpret_cast<uintptr_t>(g.b) & 15) ||
      (g.lda % 8) || (g.ldb % 8))
    return cudaErrorInvalidValue;
  const bool plain = !g.gather && !g.scatter && !g.group && g.max_ctas == 0;
  // the pair kernel also hosts copy / reduce jobs that no tile depends on
  const bool pairable = plain || (g.gather && !g.scatter && !g.group && g.max_ctas == 0 && g.gather->dep == 0 &&
                                  g.gather->n_copy_ctas % 2 == 0);
  if (g.block_n == kPairBlockN && !pairable) return cudaErrorInvalidValue;
  bool pair = g.block_n == kPairBlockN;
  if (g.block_n == 0 && pairable && pair_kernel_enabled()) {
    const long pair_tiles = static_cast<long>((g.M + 255) / 256) * ((g.N + 255) / 256);
    pair = pair_tiles >= sm_count() / 2;
  }
  if (pair) return g.out_f32 ? dispatch_pair<float>(g) : dispatch_pair<__nv_bfloat16>(g);
  if (g.block_n == kClusterSplitBlockN || (g.block_n == 0 && plain)) {
    const int split = plain ? ksplit_factor(g) : 1;
    if (g.block_n == kClusterSplitBlockN && split < 2) return cudaErrorInvalidValue;
    if (split >= 2) return g.out_f32 ? launch_ksplit<float>(g, split) : launch_ksplit<__nv_bfloat16>(g, split);
  }
  const int bn = g.block_n > 0 ? g.block_n : gemm_pick_bn(g.M, g.N);
  if (bn == 256) {
    return g.out_f32 ? dispatch_layout<256, float>(g) : dispatch_layout<256, __nv_bfloat16>(g);
  }
  if (bn == 64) {
    return g.out_f32 ? dispatch_layout<64, float>(g) : dispatch_layout<64, __nv_bfloat16>(g);
  }
  return g.out_f32 ? dispatch_layout<128, float>(g) : dispatch_layout<128, __nv_bfloat16>(g);
}

}  // namespace hb
