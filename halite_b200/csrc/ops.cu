// Memory-bound kernels of the training / RL path for sm_100a: RMSNorm, RoPE, gated
// activations, row-wise cross entropy (+entropy, z-loss, in-place gradient), fused AdamW,
// norms / casts and the GAE scan. All use 16-byte vector accesses where alignment allows
// and fp32 math; each has a plain PyTorch oracle in the Python package.
#include <cuda_bf16.h>
#include <math.h>

#include "ops.h"

namespace hb {

namespace {

// Eight bf16 values as one 16-byte word. The member is a plain uint4 so that copying the struct
// is a single 128-bit load or store (a struct of __nv_bfloat162 members is copied member by member:
// four 32-bit accesses, four times the load/store wavefronts for the same bytes).
struct alignas(16) bf16x8 {
  uint4 u;
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float (&f)[8]) {
  const uint32_t w[4] = {p.u.x, p.u.y, p.u.z, p.u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);              // low half: element 2i
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);  // high half: element 2i + 1
  }
}
__device__ __forceinline__ bf16x8 pack8(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&t);
  }
  bf16x8 p;
  p.u = make_uint4(w[0], w[1], w[2], w[3]);
  return p;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// block-wide sum, result broadcast to all threads. `red` is >= 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = (lane < (blockDim.x + 31) / 32) ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = (lane < (blockDim.x + 31) / 32) ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// ------------------------------------------------------------------ RMSNorm
constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;  // register-resident up to dim = 256 * 8 * 4 = 8192

template <bool HAS_RES, bool WRITE_H>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int dim,
                   float eps, float w_offset) {
  __shared__ float red[33];
  const long row = blockIdx.x;
  const int nvec = dim >> 3;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * dim);
  const bf16x8* rr = HAS_RES ? reinterpret_cast<const bf16x8*>(res + row * dim) : nullptr;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * dim);
  bf16x8* hr = WRITE_H ? reinterpret_cast<bf16x8*>(h_out + row * dim) : nullptr;

  float h[kNormMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      unpack8(xr[v], h[i]);
      if (HAS_RES) {
        float r[8];
        unpack8(rr[v], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) h[i][j] += r[j];
      }
      if (WRITE_H) {
        bf16x8 hp = pack8(h[i]);
        hr[v] = hp;
        // the normalisation sees the rounded residual stream, like the unfused path
        unpack8(hp, h[i]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += h[i][j] * h[i][j];
    }
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / dim + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      float wv[8], o[8];
      unpack8(wr[v], wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = h[i][j] * rstd * (wv[j] + w_offset);
      yr[v] = pack8(o);
    }
  }
}

// Backward, split in two bandwidth-shaped kernels.
// (1) dx: one warp per row (no block-level sync); the row is read twice, the second time from L1.
template <bool HAS_DRES>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                      const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                      const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                      int rows, int dim, float w_offset) {
  const int lane = threadIdx.x & 31;
  const long row = static_cast<long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = dim >> 3;
  const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + row * dim);
  const bf16x8* hr = reinterpret_cast<const bf16x8*>(h + row * dim);
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  const float rs = rstd[row];
  float dot = 0.f;
  for (int v = lane; v < nvec; v += 32) {
    float d[8], hv[8], wv[8];
    unpack8(dyr[v], d);
    unpack8(hr[v], hv);
    unpack8(wr[v], wv);
#pragma unroll
    for (int j = 0; j < 8; ++j) dot += d[j] * (wv[j] + w_offset) * hv[j];
  }
  dot = warp_sum(dot) * rs / dim;  // mean(g * xhat)
  bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + row * dim);
  const bf16x8* drr = HAS_DRES ? reinterpret_cast<const bf16x8*>(dres + row * dim) : nullptr;
  for (int v = lane; v < nvec; v += 32) {
    float d[8], hv[8], wv[8], o[8];
    unpack8(dyr[v], d);
    unpack8(hr[v], hv);
    unpack8(wr[v], wv);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = rs * (d[j] * (wv[j] + w_offset) - hv[j] * rs * dot);
    if (HAS_DRES) {
      float r[8];
      unpack8(drr[v], r);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] += r[j];
    }
    dxr[v] = pack8(o);
  }
}

// Row-in-registers variants: one 128-thread CTA per row, each thread holding VPT 16-byte vectors
// of the row (and of its companion operand) packed in registers between the reduction and the
// output pass; all loads of a row are issued before the first use, and the many small CTAs per
// SM overlap one another's load, reduce and store phases. Covers dim <= 128 * 8 * VPT.
constexpr int kRowThreads = 128;

__device__ __forceinline__ float row_sum(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  return red[0] + red[1] + red[2] + red[3];
}

template <int VPT, bool HAS_RES, bool WRITE_H>
__global__ void __launch_bounds__(kRowThreads)
rmsnorm_fwd_row_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                       __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int dim, float eps,
                       float w_offset) {
  __shared__ float red[4];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // a dependent launch may set itself up under this kernel
  const long row = blockIdx.x;
  const int nvec = dim >> 3;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * dim);
  const bf16x8* rr = HAS_RES ? reinterpret_cast<const bf16x8*>(res + row * dim) : nullptr;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8 xv[VPT], rv[HAS_RES ? VPT : 1];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * kRowThreads;
    if (v < nvec) {
      xv[i] = xr[v];
      if (HAS_RES) rv[i] = rr[v];
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * kRowThreads;
    if (v < nvec) {
      float h[8];
      unpack8(xv[i], h);
      if (HAS_RES) {
        float r[8];
        unpack8(rv[i], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] += r[j];
        xv[i] = pack8(h);          // the normalisation sees the rounded residual stream
        unpack8(xv[i], h);
        if (WRITE_H) reinterpret_cast<bf16x8*>(h_out + row * dim)[v] = xv[i];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += h[j] * h[j];
    }
  }
  ss = row_sum(ss, red);
  const float rstd = rsqrtf(ss / dim + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * dim);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * kRowThreads;
    if (v < nvec) {
      float h[8], wv[8], o[8];
      unpack8(xv[i], h);
      unpack8(wr[v], wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = h[j] * rstd * (wv[j] + w_offset);
      yr[v] = pack8(o);
    }
  }
}

template <int VPT, bool HAS_DRES>
__global__ void __launch_bounds__(kRowThreads)
rmsnorm_bwd_dx_row_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                          const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                          const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx, int dim,
                          float w_offset) {
  __shared__ float red[4];
  const long row = blockIdx.x;
  const int nvec = dim >> 3;
  const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + row * dim);
  const bf16x8* hr = reinterpret_cast<const bf16x8*>(h + row * dim);
  const bf16x8* drr = HAS_DRES ? reinterpret_cast<const bf16x8*>(dres + row * dim) : nullptr;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8 gv[VPT], hv[VPT], rv[HAS_DRES ? VPT : 1];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * kRowThreads;
    if (v < nvec) {
      gv[i] = dyr[v];
      hv[i] = hr[v];
      if (HAS_DRES) rv[i] = drr[v];
    }
  }
  const float rs = rstd[row];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * kRowThreads;
    if (v < nvec) {
      float d[8], hh[8], wv[8];
      unpack8(gv[i], d);
      unpack8(hv[i], hh);
      unpack8(wr[v], wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += d[j] * (wv[j] + w_offset) * hh[j];
    }
  }
  dot = row_sum(dot, red) * rs / dim;  // mean(g * xhat)
  bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + row * dim);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * kRowThreads;
    if (v < nvec) {
      float d[8], hh[8], wv[8], o[8];
      unpack8(gv[i], d);
      unpack8(hv[i], hh);
      unpack8(wr[v], wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rs * (d[j] * (wv[j] + w_offset) - hh[j] * rs * dot);
      if (HAS_DRES) {
        float r[8];
        unpack8(rv[i], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += r[j];
      }
      dxr[v] = pack8(o);
    }
  }
}

// (2) dw partials: CTA (x, y) sums dy * h * rstd over its row slice for 256 columns.
__global__ void __launch_bounds__(256)
rmsnorm_bwd_dw_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                      const float* __restrict__ rstd, float* __restrict__ dw_partial, int rows,
                      int dim) {
  __shared__ float red[8][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + lane * 8;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (col < dim) {
    for (long r = static_cast<long>(blockIdx.y) * 8 + warp; r < rows; r += static_cast<long>(gridDim.y) * 8) {
      float d[8], hv[8];
      unpack8(*reinterpret_cast<const bf16x8*>(dy + r * dim + col), d);
      unpack8(*reinterpret_cast<const bf16x8*>(h + r * dim + col), hv);
      const float rs = rstd[r];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += d[j] * hv[j] * rs;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[warp][lane * 8 + j] = acc[j];
  __syncthreads();
  const int c = threadIdx.x;
  if (blockIdx.x * 256 + c < dim) {
    float s = 0.f;
#pragma unroll
    for (int wi = 0; wi < 8; ++wi) s += red[wi][c];
    dw_partial[static_cast<long>(blockIdx.y) * dim + blockIdx.x * 256 + c] = s;
  }
}

__global__ void colsum_kernel(const float* __restrict__ p, int prows, int dim, void* out,
                              bool out_bf16, bool accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= dim) return;
  float s = 0.f;
  for (int r = 0; r < prows; ++r) s += p[static_cast<long>(r) * dim + c];
  if (out_bf16) {
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
    if (accumulate) s += __bfloat162float(o[c]);
    o[c] = __float2bfloat16_rn(s);
  } else {
    float* o = static_cast<float*>(out);
    if (accumulate) s += o[c];
    o[c] = s;
  }
}

// ------------------------------------------------------------------ RoPE
template <typename PosT>
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, const PosT* __restrict__ pos,
                            int tokens, int heads, int head_dim, int rot_dim, long token_stride,
                            bool interleaved, float sign) {
  // one thread per (token, head, pair-of-pairs): handles 2 rotation pairs -> 4 elements
  const int half = rot_dim >> 1;
  const int pairs2 = half >> 1;  // groups of two pairs
  const long total = static_cast<long>(tokens) * heads * pairs2;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const int pp = idx % pairs2;
    const long th = idx / pairs2;
    const int hd = th % heads;
    const long t = th / heads;
    const long p = static_cast<long>(pos[t]);
    const int i0 = pp * 2;
    const float2 c = *reinterpret_cast<const float2*>(cos_t + p * half + i0);
    float2 s = *reinterpret_cast<const float2*>(sin_t + p * half + i0);
    s.x *= sign;
    s.y *= sign;
    __nv_bfloat16* base = x + t * token_stride + static_cast<long>(hd) * head_dim;
    if (interleaved) {
      // elements (2 i0, 2 i0 + 1), (2 i0 + 2, 2 i0 + 3): one 8-byte access
      uint2* q = reinterpret_cast<uint2*>(base + 2 * i0);
      uint2 raw = *q;
      float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw.x));
      float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw.y));
      __nv_bfloat162 ra = __floats2bfloat162_rn(a.x * c.x - a.y * s.x, a.x * s.x + a.y * c.x);
      __nv_bfloat162 rb = __floats2bfloat162_rn(b.x * c.y - b.y * s.y, b.x * s.y + b.y * c.y);
      raw.x = *reinterpret_cast<uint32_t*>(&ra);
      raw.y = *reinterpret_cast<uint32_t*>(&rb);
      *q = raw;
    } else {
      __nv_bfloat162* lo = reinterpret_cast<__nv_bfloat162*>(base + i0);
      __nv_bfloat162* hi = reinterpret_cast<__nv_bfloat162*>(base + half + i0);
      float2 a = __bfloat1622float2(*lo);
      float2 b = __bfloat1622float2(*hi);
      *lo = __floats2bfloat162_rn(a.x * c.x - b.x * s.x, a.y * c.y - b.y * s.y);
      *hi = __floats2bfloat162_rn(b.x * c.x + a.x * s.x, b.y * c.y + a.y * s.y);
    }
  }
}

// 16-byte variant, optionally out of place (src and dst may have different token strides, e.g.
// a contiguous gradient rotated into its slot of a packed qkv gradient). One thread per
// (token, group of `hpt` heads, 8 elements): the thread reads its slice of the token's cos/sin row
// once and walks the heads of its group with it (hpt = 1: one thread per head; hpt = heads: the
// tables are read once per token instead of once per head). Elements past rot_dim are copied when
// src != dst.
template <typename PosT, bool INTERLEAVED>
__global__ void rope_vec_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                const PosT* __restrict__ pos, int tokens, int heads, int head_dim,
                                int rot_dim, long src_stride, long dst_stride, float sign, bool in_place,
                                int hpt) {
  const int half = rot_dim >> 1;
  const int vph = head_dim >> 3;
  const int groups = (heads + hpt - 1) / hpt;
  const long total = static_cast<long>(tokens) * groups * vph;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const int j = idx % vph;
    const long tg = idx / vph;
    const int h0 = (tg % groups) * hpt;
    const int h1 = min(heads, h0 + hpt);
    const long t = tg / groups;
    const __nv_bfloat16* s = src + t * src_stride + 8 * j;
    __nv_bfloat16* d = dst + t * dst_stride + 8 * j;
    if (INTERLEAVED) {
      if (8 * j < rot_dim) {
        const long p = static_cast<long>(pos[t]);
        const float4 c = *reinterpret_cast<const float4*>(cos_t + p * half + 4 * j);
        const float4 sn = *reinterpret_cast<const float4*>(sin_t + p * half + 4 * j);
        const float cc[4] = {c.x, c.y, c.z, c.w};
        const float ss[4] = {sn.x * sign, sn.y * sign, sn.z * sign, sn.w * sign};
#pragma unroll 4
        for (int hd = h0; hd < h1; ++hd) {
          float f[8], o[8];
          unpack8(*reinterpret_cast<const bf16x8*>(s + static_cast<long>(hd) * head_dim), f);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            o[2 * k] = f[2 * k] * cc[k] - f[2 * k + 1] * ss[k];
            o[2 * k + 1] = f[2 * k] * ss[k] + f[2 * k + 1] * cc[k];
          }
          *reinterpret_cast<bf16x8*>(d + static_cast<long>(hd) * head_dim) = pack8(o);
        }
      } else if (!in_place) {
#pragma unroll 4
        for (int hd = h0; hd < h1; ++hd)
          *reinterpret_cast<bf16x8*>(d + static_cast<long>(hd) * head_dim) =
              *reinterpret_cast<const bf16x8*>(s + static_cast<long>(hd) * head_dim);
      }
    } else {
      const int hv = half >> 3;
      if (j < hv) {
        const long p = static_cast<long>(pos[t]);
        float cc[8], ss[8];
        *reinterpret_cast<float4*>(cc) = *reinterpret_cast<const float4*>(cos_t + p * half + 8 * j);
        *reinterpret_cast<float4*>(cc + 4) = *reinterpret_cast<const float4*>(cos_t + p * half + 8 * j + 4);
        *reinterpret_cast<float4*>(ss) = *reinterpret_cast<const float4*>(sin_t + p * half + 8 * j);
        *reinterpret_cast<float4*>(ss + 4) = *reinterpret_cast<const float4*>(sin_t + p * half + 8 * j + 4);
#pragma unroll
        for (int k = 0; k < 8; ++k) ss[k] *= sign;
#pragma unroll 2
        for (int hd = h0; hd < h1; ++hd) {
          const long off = static_cast<long>(hd) * head_dim;
          float lo[8], hi[8], olo[8], ohi[8];
          unpack8(*reinterpret_cast<const bf16x8*>(s + off), lo);
          unpack8(*reinterpret_cast<const bf16x8*>(s + off + half), hi);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            olo[k] = lo[k] * cc[k] - hi[k] * ss[k];
            ohi[k] = hi[k] * cc[k] + lo[k] * ss[k];
          }
          *reinterpret_cast<bf16x8*>(d + off) = pack8(olo);
          *reinterpret_cast<bf16x8*>(d + off + half) = pack8(ohi);
        }
      } else if (8 * j >= rot_dim && !in_place) {
#pragma unroll 4
        for (int hd = h0; hd < h1; ++hd)
          *reinterpret_cast<bf16x8*>(d + static_cast<long>(hd) * head_dim) =
              *reinterpret_cast<const bf16x8*>(s + static_cast<long>(hd) * head_dim);
      }
    }
  }
}

// ------------------------------------------------------------------ gated activation
__device__ __forceinline__ float act_fwd(float g, int kind) {
  if (kind == 0) return g / (1.f + __expf(-g));
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * g * (1.f + tanhf(k0 * (g + k1 * g * g * g)));
}
__device__ __forceinline__ float act_grad(float g, int kind) {
  if (kind == 0) {
    const float s = 1.f / (1.f + __expf(-g));
    return s * (1.f + g * (1.f - s));
  }
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float t = tanhf(k0 * (g + k1 * g * g * g));
  return 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * k0 * (1.f + 3.f * k1 * g * g);
}

// Tensors are [rows, row] with independent leading dimensions, so gate/up may be the two
// halves of one fused projection output.
__global__ void gated_fwd_kernel(const __nv_bfloat16* __restrict__ gate,
                                 const __nv_bfloat16* __restrict__ up,
                                 __nv_bfloat16* __restrict__ out, long nvec, int row_vec,
                                 long gate_ld, long up_ld, int kind) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // a dependent launch may set itself up under this kernel
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / row_vec;
    const int c = (i - r * row_vec) * 8;
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const bf16x8*>(gate + r * gate_ld + c), g);
    unpack8(*reinterpret_cast<const bf16x8*>(up + r * up_ld + c), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = act_fwd(g[j], kind) * u[j];
    *reinterpret_cast<bf16x8*>(out + r * static_cast<long>(row_vec) * 8 + c) = pack8(o);
  }
}

__global__ void gated_bwd_kernel(const __nv_bfloat16* __restrict__ gate,
                                 const __nv_bfloat16* __restrict__ up,
                                 const __nv_bfloat16* __restrict__ dout,
                                 __nv_bfloat16* __restrict__ dgate, __nv_bfloat16* __restrict__ dup,
                                 long nvec, int row_vec, long gate_ld, long up_ld, long dgate_ld,
                                 long dup_ld, int kind) {
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / row_vec;
    const int c = (i - r * row_vec) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const bf16x8*>(gate + r * gate_ld + c), g);
    unpack8(*reinterpret_cast<const bf16x8*>(up + r * up_ld + c), u);
    unpack8(*reinterpret_cast<const bf16x8*>(dout + r * static_cast<long>(row_vec) * 8 + c), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dg[j] = d[j] * u[j] * act_grad(g[j], kind);
      du[j] = d[j] * act_fwd(g[j], kind);
    }
    *reinterpret_cast<bf16x8*>(dgate + r * dgate_ld + c) = pack8(dg);
    *reinterpret_cast<bf16x8*>(dup + r * dup_ld + c) = pack8(du);
  }
}

// ------------------------------------------------------------------ cross entropy
constexpr int kCEThreads = 1024;

template <typename T>
__device__ __forceinline__ float ld_logit(const T* p, long i);
template <>
__device__ __forceinline__ float ld_logit<float>(const float* p, long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, long i) {
  return __bfloat162float(p[i]);
}
template <typename T>
__device__ __forceinline__ void st_logit(T* p, long i, float v);
template <>
__device__ __forceinline__ void st_logit<float>(float* p, long i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void st_logit<__nv_bfloat16>(__nv_bfloat16* p, long i, float v) {
  p[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float cap(float x, float scale, float softcap) {
  x *= scale;
  if (softcap > 0.f) x = softcap * tanhf(x / softcap);
  return x;
}

// One CTA per row. Pass 1: online (max, sum exp, sum x*exp) over the vocabulary slice.
// Pass 2 (optional): gradient written over the row.
template <typename T>
__global__ void __launch_bounds__(kCEThreads)
ce_kernel(CEArgs a) {
  __shared__ float red[33];
  const long row = blockIdx.x;
  const T* lg = static_cast<const T*>(a.logits) + row * a.ld;
  T* dl = a.dlogits ? static_cast<T*>(a.dlogits) + row * a.ld : nullptr;
  const int64_t tgt = a.targets ? a.targets[row] : a.ignore_index;
  const bool ignored = (tgt == a.ignore_index);
  const float scale = a.logit_scale * (a.row_scale ? a.row_scale[row] : 1.f);
  const int V = a.vocab;

  // vectorised pass 1: 8 bf16 / 4 fp32 per access when the row start is 16-byte aligned
  float m = -INFINITY, s = 0.f, sx = 0.f, sumx = 0.f;
  constexpr int VEC = 16 / sizeof(T);
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(lg) & 15) == 0);
  const int nv = vec_ok ? V / VEC : 0;
  for (int v = threadIdx.x; v < nv; v += kCEThreads) {
    float f[VEC];
    if constexpr (sizeof(T) == 2) {
      float t8[8];
      unpack8(reinterpret_cast<const bf16x8*>(lg)[v], t8);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = t8[j];
    } else {
      float4 t4 = reinterpret_cast<const float4*>(lg)[v];
      f[0] = t4.x; f[1] = t4.y; f[2] = t4.z; f[3] = t4.w;
    }
    float lm = -INFINITY;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      f[j] = cap(f[j], scale, a.softcap);
      lm = fmaxf(lm, f[j]);
    }
    if (lm > m) {
      const float r = __expf(m - lm);
      s *= r;
      sx *= r;
      m = lm;
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float e = __expf(f[j] - m);
      s += e;
      sx += e * f[j];
      sumx += f[j];
    }
  }
  for (int i = nv * VEC + threadIdx.x; i < V; i += kCEThreads) {
    const float x = cap(ld_logit<T>(lg, i), scale, a.softcap);
    if (x > m) {
      const float r = __expf(m - x);
      s *= r;
      sx *= r;
      m = x;
    }
    const float e = __expf(x - m);
    s += e;
    sx += e * x;
    sumx += x;
  }
  const float gm = block_max(m, red);
  const float r = (m == -INFINITY) ? 0.f : __expf(m - gm);
  s = block_sum(s * r, red);
  sx = block_sum(sx * r, red);
  if (a.label_smoothing > 0.f) sumx = block_sum(sumx, red);
  const float lse = gm + logf(s);

  float xt = 0.f;
  const long tl = static_cast<long>(tgt) - a.vocab_start;
  const bool own_target = !ignored && tl >= 0 && tl < V;
  if (own_target) xt = cap(ld_logit<T>(lg, tl), scale, a.softcap);

  if (threadIdx.x == 0) {
    if (a.lse) a.lse[row] = lse;
    if (a.entropy) a.entropy[row] = lse - sx / s;  // H = lse - E[x]
    float loss = 0.f, z = 0.f;
    if (!ignored) {
      loss = lse - xt;
      if (a.label_smoothing > 0.f) {
        const float smooth = lse - sumx / V;
        loss = (1.f - a.label_smoothing) * loss + a.label_smoothing * smooth;
      }
      z = a.z_loss * lse * lse;
      loss += z;
    }
    if (a.loss) a.loss[row] = loss;
    if (a.zloss) a.zloss[row] = z;
  }
  if (!dl) return;

  float gs = a.grad_scale * (a.grad_scale_ptr ? *a.grad_scale_ptr : 1.f);
  if (ignored) gs = 0.f;
  const float pz = 1.f + 2.f * a.z_loss * lse;
  const float eps_ls = a.label_smoothing;
  auto grad_of = [&](float raw_logit, int i) {
    const float raw = raw_logit * scale;
    float x = raw, dcap = 1.f;
    if (a.softcap > 0.f) {
      const float t = tanhf(raw / a.softcap);
      x = a.softcap * t;
      dcap = 1.f - t * t;
    }
    const float p = __expf(x - lse);
    float g = p * pz - eps_ls / V;
    if (i == tl && own_target) g -= (1.f - eps_ls);
    return g * gs * dcap * scale;
  };
  const bool vec2 = vec_ok && ((reinterpret_cast<uintptr_t>(dl) & 15) == 0);
  const int nv2 = vec2 ? V / VEC : 0;
  for (int v = threadIdx.x; v < nv2; v += kCEThreads) {
    if constexpr (sizeof(T) == 2) {
      float f[8];
      unpack8(reinterpret_cast<const bf16x8*>(lg)[v], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = grad_of(f[j], v * 8 + j);
      reinterpret_cast<bf16x8*>(dl)[v] = pack8(f);
    } else {
      float4 t4 = reinterpret_cast<const float4*>(lg)[v];
      t4.x = grad_of(t4.x, v * 4);
      t4.y = grad_of(t4.y, v * 4 + 1);
      t4.z = grad_of(t4.z, v * 4 + 2);
      t4.w = grad_of(t4.w, v * 4 + 3);
      reinterpret_cast<float4*>(dl)[v] = t4;
    }
  }
  for (int i = nv2 * VEC + threadIdx.x; i < V; i += kCEThreads)
    st_logit<T>(dl, i, grad_of(ld_logit<T>(lg, i), i));
}

// Backward of (log-prob of target, entropy) w.r.t. logits, one CTA per row:
//   d logit_i = scale * [ g_lp * (1[i == t] - p_i) - g_ent * p_i * (log p_i + H) ]
template <typename T>
__global__ void __launch_bounds__(kCEThreads)
logprob_entropy_bwd_kernel(LogprobBwdArgs a) {
  const long row = blockIdx.x;
  const T* lg = static_cast<const T*>(a.logits) + row * a.ld;
  T* dl = static_cast<T*>(a.dlogits) + row * a.ld;
  const float scale = a.logit_scale * (a.row_scale ? a.row_scale[row] : 1.f);
  const float lse = a.lse[row];
  const float H = a.entropy ? a.entropy[row] : 0.f;
  const int64_t tgt = a.targets[row];
  const bool ignored = (tgt == a.ignore_index);
  const float glp = (a.g_logprob && !ignored) ? a.g_logprob[row] : 0.f;
  const float gen = a.g_entropy ? a.g_entropy[row] : 0.f;
  const long tl = static_cast<long>(tgt) - a.vocab_start;
  for (int i = threadIdx.x; i < a.vocab; i += kCEThreads) {
    const float x = ld_logit<T>(lg, i) * scale;
    const float logp = x - lse;
    const float p = __expf(logp);
    float g = -glp * p - gen * p * (logp + H);
    if (i == tl) g += glp;
    st_logit<T>(dl, i, g * scale);
  }
}

// ------------------------------------------------------------------ AdamW / norms / casts
template <bool GRAD_F32>
__global__ void adamw_kernel(AdamWArgs a, float bc1, float bc2) {
  const float gsc = a.grad_scale * (a.grad_scale_ptr ? *a.grad_scale_ptr : 1.f);
  const long n4 = a.n >> 2;
  __nv_bfloat16* pb = static_cast<__nv_bfloat16*>(a.param_bf16);
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float4 p = reinterpret_cast<float4*>(a.master)[i];
    float4 m = reinterpret_cast<float4*>(a.exp_avg)[i];
    float4 v = reinterpret_cast<float4*>(a.exp_avg_sq)[i];
    float g[4];
    if (GRAD_F32) {
      float4 t = reinterpret_cast<const float4*>(a.grad)[i];
      g[0] = t.x; g[1] = t.y; g[2] = t.z; g[3] = t.w;
    } else {
      uint2 t = reinterpret_cast<const uint2*>(a.grad)[i];
      float2 lo = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&t.x));
      float2 hi = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&t.y));
      g[0] = lo.x; g[1] = lo.y; g[2] = hi.x; g[3] = hi.y;
    }
    float* pp = reinterpret_cast<float*>(&p);
    float* mm = reinterpret_cast<float*>(&m);
    float* vv = reinterpret_cast<float*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = g[j] * gsc;
      pp[j] *= (1.f - a.lr * a.weight_decay);
      mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gj;
      vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gj * gj;
      const float denom = sqrtf(vv[j]) / bc2 + a.eps;  // bc2 = sqrt(1 - beta2^t)
      pp[j] -= (a.lr / bc1) * (mm[j] / denom);
    }
    reinterpret_cast<float4*>(a.master)[i] = p;
    reinterpret_cast<float4*>(a.exp_avg)[i] = m;
    reinterpret_cast<float4*>(a.exp_avg_sq)[i] = v;
    if (pb) {
      uint2 o;
      __nv_bfloat162 lo = __floats2bfloat162_rn(pp[0], pp[1]);
      __nv_bfloat162 hi = __floats2bfloat162_rn(pp[2], pp[3]);
      o.x = *reinterpret_cast<uint32_t*>(&lo);
      o.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(pb)[i] = o;
    }
  }
  // tail (n not a multiple of 4)
  if (blockIdx.x == 0 && threadIdx.x < (a.n & 3)) {
    const long i = (n4 << 2) + threadIdx.x;
    float gj = (GRAD_F32 ? static_cast<const float*>(a.grad)[i]
                         : __bfloat162float(static_cast<const __nv_bfloat16*>(a.grad)[i])) * gsc;
    float p = a.master[i] * (1.f - a.lr * a.weight_decay);
    float m = a.beta1 * a.exp_avg[i] + (1.f - a.beta1) * gj;
    float v = a.beta2 * a.exp_avg_sq[i] + (1.f - a.beta2) * gj * gj;
    p -= (a.lr / bc1) * (m / (sqrtf(v) / bc2 + a.eps));
    a.master[i] = p; a.exp_avg[i] = m; a.exp_avg_sq[i] = v;
    if (pb) pb[i] = __float2bfloat16_rn(p);
  }
}

template <bool F32>
__global__ void sumsq_kernel(const void* __restrict__ x, long n, float* __restrict__ out) {
  __shared__ float red[33];
  float acc = 0.f;
  if (F32) {
    const float4* p = static_cast<const float4*>(x);
    const long n4 = n >> 2;
    for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n4;
         i += static_cast<long>(gridDim.x) * blockDim.x) {
      float4 t = p[i];
      acc += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
      float t = static_cast<const float*>(x)[(n4 << 2) + threadIdx.x];
      acc += t * t;
    }
  } else {
    const bf16x8* p = static_cast<const bf16x8*>(x);
    const long n8 = n >> 3;
    for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8;
         i += static_cast<long>(gridDim.x) * blockDim.x) {
      float f[8];
      unpack8(p[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += f[j] * f[j];
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
      float t = __bfloat162float(static_cast<const __nv_bfloat16*>(x)[(n8 << 3) + threadIdx.x]);
      acc += t * t;
    }
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) atomicAdd(out, acc);
}

__global__ void clip_coef_kernel(const float* sumsq, float max_norm, float* out) {
  const float norm = sqrtf(sumsq[0]);
  out[0] = (max_norm > 0.f) ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
  out[1] = norm;
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ s, __nv_bfloat16* __restrict__ d,
                                   long n) {
  const long n4 = n >> 2;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float4 t = reinterpret_cast<const float4*>(s)[i];
    uint2 o;
    __nv_bfloat162 lo = __floats2bfloat162_rn(t.x, t.y);
    __nv_bfloat162 hi = __floats2bfloat162_rn(t.z, t.w);
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    reinterpret_cast<uint2*>(d)[i] = o;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const long i = (n4 << 2) + threadIdx.x;
    d[i] = __float2bfloat16_rn(s[i]);
  }
}

__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ s, float* __restrict__ d,
                                   long n, float scale, bool accumulate) {
  const long n4 = n >> 2;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    uint2 t = reinterpret_cast<const uint2*>(s)[i];
    float2 lo = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&t.x));
    float2 hi = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&t.y));
    float4 o = make_float4(lo.x * scale, lo.y * scale, hi.x * scale, hi.y * scale);
    if (accumulate) {
      float4 old = reinterpret_cast<float4*>(d)[i];
      o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
    }
    reinterpret_cast<float4*>(d)[i] = o;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const long i = (n4 << 2) + threadIdx.x;
    float o = __bfloat162float(s[i]) * scale;
    if (accumulate) o += d[i];
    d[i] = o;
  }
}

// ------------------------------------------------------------------ GAE
// One thread per sequence; the T-long reverse recurrence is inherently serial per row.
__global__ void gae_kernel(const float* __restrict__ rewards, const float* __restrict__ values,
                           const float* __restrict__ mask, float* __restrict__ adv,
                           float* __restrict__ ret, int B, int T, float gamma, float lam) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const long o = static_cast<long>(b) * T;
  float last = 0.f, next_v = 0.f;
  for (int t = T - 1; t >= 0; --t) {
    const float mk = mask ? mask[o + t] : 1.f;
    const float v = values[o + t];
    const float delta = rewards[o + t] + gamma * next_v - v;
    const float cur = delta + gamma * lam * last;
    // positions outside the response keep the running state untouched
    last = mk * cur + (1.f - mk) * last;
    next_v = mk * v + (1.f - mk) * next_v;
    adv[o + t] = mk * cur;
    ret[o + t] = mk * (cur + v);
  }
}

int grid_for(long work_items, int threads, int max_blocks = 148 * 16) {
  long b = (work_items + threads - 1) / threads;
  if (b > max_blocks) b = max_blocks;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace

// ------------------------------------------------------------------ launchers
cudaError_t rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* h_out,
                        float* rstd, int rows, int dim, float eps, float w_offset,
                        cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  if (dim % 8 != 0 || dim > kNormThreads * 8 * kNormMaxVec) return cudaErrorInvalidValue;
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto R = static_cast<const __nv_bfloat16*>(residual);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto Y = static_cast<__nv_bfloat16*>(y);
  auto H = static_cast<__nv_bfloat16*>(h_out);
  const int vpt = (dim / 8 + kRowThreads - 1) / kRowThreads;
  if (vpt <= 8) {
#define HB_NORM_FWD(V)                                                                                        \
  do {                                                                                                        \
    if (R && H)                                                                                               \
      rmsnorm_fwd_row_kernel<V, true, true><<<rows, kRowThreads, 0, stream>>>(X, R, W, Y, H, rstd, dim, eps, w_offset);  \
    else if (R)                                                                                               \
      rmsnorm_fwd_row_kernel<V, true, false><<<rows, kRowThreads, 0, stream>>>(X, R, W, Y, H, rstd, dim, eps, w_offset); \
    else                                                                                                      \
      rmsnorm_fwd_row_kernel<V, false, false><<<rows, kRowThreads, 0, stream>>>(X, R, W, Y, H, rstd, dim, eps, w_offset); \
  } while (0)
    if (vpt <= 1) HB_NORM_FWD(1);
    else if (vpt <= 2) HB_NORM_FWD(2);
    else if (vpt <= 3) HB_NORM_FWD(3);
    else if (vpt <= 4) HB_NORM_FWD(4);
    else if (vpt <= 6) HB_NORM_FWD(6);
    else HB_NORM_FWD(8);
#undef HB_NORM_FWD
    return cudaGetLastError();
  }
  if (R && H)
    rmsnorm_fwd_kernel<true, true><<<rows, kNormThreads, 0, stream>>>(X, R, W, Y, H, rstd, dim, eps, w_offset);
  else if (R)
    rmsnorm_fwd_kernel<true, false><<<rows, kNormThreads, 0, stream>>>(X, R, W, Y, H, rstd, dim, eps, w_offset);
  else
    rmsnorm_fwd_kernel<false, false><<<rows, kNormThreads, 0, stream>>>(X, R, W, Y, H, rstd, dim, eps, w_offset);
  return cudaGetLastError();
}

cudaError_t rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd,
                        const void* dres, void* dx, float* dw_partial, int partial_rows, int rows,
                        int dim, float w_offset, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  if (dim % 8 != 0 || dim > kNormThreads * 8 * kNormMaxVec || partial_rows < 1)
    return cudaErrorInvalidValue;
  auto DY = static_cast<const __nv_bfloat16*>(dy);
  auto H = static_cast<const __nv_bfloat16*>(h);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto DR = static_cast<const __nv_bfloat16*>(dres);
  auto DX = static_cast<__nv_bfloat16*>(dx);
  const int grid_dx = static_cast<int>((static_cast<long long>(rows) + 7) / 8);   // rows may be near 2^31
  const int vpt = (dim / 8 + kRowThreads - 1) / kRowThreads;
#define HB_NORM_BWD(V)                                                                                          \
  do {                                                                                                          \
    if (DR)                                                                                                     \
      rmsnorm_bwd_dx_row_kernel<V, true><<<rows, kRowThreads, 0, stream>>>(DY, H, W, rstd, DR, DX, dim, w_offset);  \
    else                                                                                                        \
      rmsnorm_bwd_dx_row_kernel<V, false><<<rows, kRowThreads, 0, stream>>>(DY, H, W, rstd, DR, DX, dim, w_offset); \
  } while (0)
  if (vpt <= 1) HB_NORM_BWD(1);
  else if (vpt <= 2) HB_NORM_BWD(2);
  else if (vpt <= 3) HB_NORM_BWD(3);
  else if (vpt <= 4) HB_NORM_BWD(4);
  else if (vpt <= 6) HB_NORM_BWD(6);
  else if (vpt <= 8) HB_NORM_BWD(8);
  else if (DR)
    rmsnorm_bwd_dx_kernel<true><<<grid_dx, 256, 0, stream>>>(DY, H, W, rstd, DR, DX, rows, dim, w_offset);
  else
    rmsnorm_bwd_dx_kernel<false><<<grid_dx, 256, 0, stream>>>(DY, H, W, rstd, DR, DX, rows, dim, w_offset);
#undef HB_NORM_BWD
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  // every one of the `partial_rows` rows is written (row slices may be empty -> zeros)
  dim3 grid_dw((dim + 255) / 256, partial_rows);
  rmsnorm_bwd_dw_kernel<<<grid_dw, 256, 0, stream>>>(DY, H, rstd, dw_partial, rows, dim);
  return cudaGetLastError();
}

cudaError_t colsum_f32(const float* partial, int prows, int dim, void* out, bool out_bf16,
                       bool accumulate, cudaStream_t stream) {
  colsum_kernel<<<(dim + 255) / 256, 256, 0, stream>>>(partial, prows, dim, out, out_bf16, accumulate);
  return cudaGetLastError();
}

cudaError_t rope_apply(const void* src, void* dst, const float* cos, const float* sin, const void* positions,
                       bool pos_is_i64, int tokens, int heads, int head_dim, int rot_dim, long src_stride,
                       long dst_stride, bool interleaved, bool conjugate, cudaStream_t stream) {
  if (tokens == 0 || heads == 0) return cudaSuccess;
  const bool in_place = src == dst && src_stride == dst_stride;
  if (rot_dim > head_dim) return cudaErrorInvalidValue;
  const float sign = conjugate ? -1.f : 1.f;
  const bool aligned = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) |
                         reinterpret_cast<uintptr_t>(cos) | reinterpret_cast<uintptr_t>(sin)) & 15) == 0;
  const bool vec_ok = aligned && head_dim % 8 == 0 && src_stride % 8 == 0 && dst_stride % 8 == 0 &&
                      rot_dim % (interleaved ? 8 : 16) == 0;
  auto S = static_cast<const __nv_bfloat16*>(src);
  auto D = static_cast<__nv_bfloat16*>(dst);
  if (vec_ok) {
    // enough tokens to fill the GPU with one thread per (token, 8 elements): that thread walks all
    // heads with one read of the tables; otherwise one thread per head
    const int hpt = static_cast<long>(tokens) * (head_dim / 8) >= (1L << 18) ? heads : 1;
    const long total = static_cast<long>(tokens) * ((heads + hpt - 1) / hpt) * (head_dim / 8);
    const int grid = grid_for(total, 256);
#define HB_ROPE_VEC(PT, IL)                                                                              \
  rope_vec_kernel<PT, IL><<<grid, 256, 0, stream>>>(S, D, cos, sin, static_cast<const PT*>(positions), tokens, \
                                                    heads, head_dim, rot_dim, src_stride, dst_stride, sign,    \
                                                    in_place, hpt)
    if (pos_is_i64) {
      if (interleaved) HB_ROPE_VEC(int64_t, true);
      else HB_ROPE_VEC(int64_t, false);
    } else {
      if (interleaved) HB_ROPE_VEC(int32_t, true);
      else HB_ROPE_VEC(int32_t, false);
    }
#undef HB_ROPE_VEC
    return cudaGetLastError();
  }
  // narrow fallback (rotation widths the 16-byte kernel does not cover): works in place, so an
  // out-of-place call first copies the rows over
  if (!in_place) {
    cudaError_t e = cudaMemcpy2DAsync(dst, static_cast<size_t>(dst_stride) * 2, src, static_cast<size_t>(src_stride) * 2,
                                      static_cast<size_t>(heads) * head_dim * 2, tokens, cudaMemcpyDeviceToDevice,
                                      stream);
    if (e != cudaSuccess) return e;
    if (rot_dim == 0) return cudaSuccess;
  }
  if (rot_dim % 4 != 0 || head_dim % 4 != 0 || dst_stride % 4 != 0 || rot_dim == 0)
    return cudaErrorInvalidValue;
  const long total = static_cast<long>(tokens) * heads * (rot_dim / 4);
  const int grid = grid_for(total, 256);
  if (pos_is_i64)
    rope_kernel<int64_t><<<grid, 256, 0, stream>>>(D, cos, sin, static_cast<const int64_t*>(positions), tokens, heads, head_dim, rot_dim, dst_stride, interleaved, sign);
  else
    rope_kernel<int32_t><<<grid, 256, 0, stream>>>(D, cos, sin, static_cast<const int32_t*>(positions), tokens, heads, head_dim, rot_dim, dst_stride, interleaved, sign);
  return cudaGetLastError();
}

cudaError_t rope_inplace(void* x, const float* cos, const float* sin, const void* positions,
                         bool pos_is_i64, int tokens, int heads, int head_dim, int rot_dim,
                         long token_stride, bool interleaved, bool conjugate, cudaStream_t stream) {
  return rope_apply(x, x, cos, sin, positions, pos_is_i64, tokens, heads, head_dim, rot_dim, token_stride,
                    token_stride, interleaved, conjugate, stream);
}

cudaError_t gated_act_fwd(const void* gate, const void* up, void* out, long n, long row, long gate_ld,
                          long up_ld, int kind, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  if (row % 8 || gate_ld % 8 || up_ld % 8) return cudaErrorInvalidValue;
  const long nvec = n / 8;
  gated_fwd_kernel<<<grid_for(nvec, 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up),
      static_cast<__nv_bfloat16*>(out), nvec, static_cast<int>(row / 8), gate_ld, up_ld, kind);
  return cudaGetLastError();
}

cudaError_t gated_act_bwd(const void* gate, const void* up, const void* dout, void* dgate, void* dup,
                          long n, long row, long gate_ld, long up_ld, long dgate_ld, long dup_ld,
                          int kind, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  if (row % 8 || gate_ld % 8 || up_ld % 8 || dgate_ld % 8 || dup_ld % 8) return cudaErrorInvalidValue;
  const long nvec = n / 8;
  gated_bwd_kernel<<<grid_for(nvec, 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up),
      static_cast<const __nv_bfloat16*>(dout), static_cast<__nv_bfloat16*>(dgate),
      static_cast<__nv_bfloat16*>(dup), nvec, static_cast<int>(row / 8), gate_ld, up_ld, dgate_ld,
      dup_ld, kind);
  return cudaGetLastError();
}

cudaError_t cross_entropy_fwd(const CEArgs& a, cudaStream_t stream) {
  if (a.rows == 0) return cudaSuccess;
  if (a.logits_f32)
    ce_kernel<float><<<a.rows, kCEThreads, 0, stream>>>(a);
  else
    ce_kernel<__nv_bfloat16><<<a.rows, kCEThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t logprob_entropy_bwd(const LogprobBwdArgs& a, cudaStream_t stream) {
  if (a.rows == 0) return cudaSuccess;
  if (a.logits_f32)
    logprob_entropy_bwd_kernel<float><<<a.rows, kCEThreads, 0, stream>>>(a);
  else
    logprob_entropy_bwd_kernel<__nv_bfloat16><<<a.rows, kCEThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t adamw_step(const AdamWArgs& a, cudaStream_t stream) {
  if (a.n == 0) return cudaSuccess;
  const float bc1 = 1.f - powf(a.beta1, static_cast<float>(a.step));
  const float bc2 = sqrtf(1.f - powf(a.beta2, static_cast<float>(a.step)));
  const int grid = grid_for((a.n + 3) / 4, 256);
  if (a.grad_f32)
    adamw_kernel<true><<<grid, 256, 0, stream>>>(a, bc1, bc2);
  else
    adamw_kernel<false><<<grid, 256, 0, stream>>>(a, bc1, bc2);
  return cudaGetLastError();
}

cudaError_t sumsq(const void* x, bool is_f32, long n, float* out, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  const int grid = grid_for(n / 8 + 1, 256, 148 * 4);
  if (is_f32)
    sumsq_kernel<true><<<grid, 256, 0, stream>>>(x, n, out);
  else
    sumsq_kernel<false><<<grid, 256, 0, stream>>>(x, n, out);
  return cudaGetLastError();
}

cudaError_t clip_coef(const float* ss, float max_norm, float* out, cudaStream_t stream) {
  clip_coef_kernel<<<1, 1, 0, stream>>>(ss, max_norm, out);
  return cudaGetLastError();
}

cudaError_t cast_f32_to_bf16(const float* src, void* dst, long n, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  f32_to_bf16_kernel<<<grid_for(n / 4 + 1, 256), 256, 0, stream>>>(src, static_cast<__nv_bfloat16*>(dst), n);
  return cudaGetLastError();
}

cudaError_t cast_bf16_to_f32(const void* src, float* dst, long n, float scale, bool accumulate,
                             cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  bf16_to_f32_kernel<<<grid_for(n / 4 + 1, 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(src), dst, n, scale, accumulate);
  return cudaGetLastError();
}

cudaError_t gae(const float* rewards, const float* values, const float* mask, float* adv,
                float* ret, int B, int T, float gamma, float lam, cudaStream_t stream) {
  if (B == 0 || T == 0) return cudaSuccess;
  gae_kernel<<<(B + 63) / 64, 64, 0, stream>>>(rewards, values, mask, adv, ret, B, T, gamma, lam);
  return cudaGetLastError();
}

// ---- first-order linear recurrence over a packed row -------------------------------------------
// h[t] = a[t] * h[prev] + b[t] * x[t] inside each sequence [cu[s], cu[s+1]) of a packed row, with
// h = 0 before a sequence's first step; REVERSE walks each sequence from its last token down.
// One thread owns one channel of one sequence: the recurrence is serial in t, the loads are not,
// so eight steps of x, a and b are fetched before the eight dependent FMAs run.
template <typename T> __device__ __forceinline__ float scan_load(const T* p);
template <> __device__ __forceinline__ float scan_load<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float scan_load<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __uint_as_float(static_cast<uint32_t>(__ldg(reinterpret_cast<const unsigned short*>(p))) << 16);
}

template <typename T, bool REVERSE>
__global__ void __launch_bounds__(128)
linear_scan_kernel(const T* __restrict__ x, const float* __restrict__ a, const float* __restrict__ b,
                   const int* __restrict__ cu, float* __restrict__ out, int dim) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= dim) return;
  const int lo = cu[blockIdx.y], hi = cu[blockIdx.y + 1];
  const int n = hi - lo;
  constexpr int U = 8;
  float h = 0.f;
  for (int i = 0; i < n; i += U) {
    float xv[U], av[U], bv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = i + u;
      if (k < n) {
        const int t = REVERSE ? hi - 1 - k : lo + k;
        xv[u] = scan_load(x + (long)t * dim + c);
        av[u] = __ldg(a + t);
        bv[u] = __ldg(b + t);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = i + u;
      if (k < n) {
        const int t = REVERSE ? hi - 1 - k : lo + k;
        h = fmaf(av[u], h, bv[u] * xv[u]);
        out[(long)t * dim + c] = h;
      }
    }
  }
}

cudaError_t linear_scan(const void* x, bool x_bf16, const float* a, const float* b, const int* cu_seqlens,
                        int n_seqs, int dim, bool reverse, float* out, cudaStream_t stream) {
  if (n_seqs == 0 || dim == 0) return cudaSuccess;
  if (n_seqs > 65535) return cudaErrorInvalidValue;
  const dim3 grid((dim + 127) / 128, n_seqs);
  if (x_bf16) {
    auto xp = static_cast<const __nv_bfloat16*>(x);
    if (reverse) linear_scan_kernel<__nv_bfloat16, true><<<grid, 128, 0, stream>>>(xp, a, b, cu_seqlens, out, dim);
    else linear_scan_kernel<__nv_bfloat16, false><<<grid, 128, 0, stream>>>(xp, a, b, cu_seqlens, out, dim);
  } else {
    auto xp = static_cast<const float*>(x);
    if (reverse) linear_scan_kernel<float, true><<<grid, 128, 0, stream>>>(xp, a, b, cu_seqlens, out, dim);
    else linear_scan_kernel<float, false><<<grid, 128, 0, stream>>>(xp, a, b, cu_seqlens, out, dim);
  }
  return cudaGetLastError();
}

}  // namespace hb
