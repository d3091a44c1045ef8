// Allocation-free RMSNorm backward: see rmsnorm_bwd_fixed_scratch.h for the contract.
//
// The per-slice partial sums of dw, which the regular path keeps in a tensor it asks torch for,
// live here in a file-scope device array. Its address is taken once per device through the
// runtime's symbol lookup and handed to the same kernels as a plain pointer.
#include "rmsnorm_bwd_fixed_scratch.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "ops.h"

namespace {

constexpr int kMaxDevices = 64;

// [slice][column] partial sums; a call with `dim` columns uses the first slices * dim floats
static __device__ __align__(256) float g_dw_slices[HB_RMSNORM_BWD_FIXED_SLICES * HB_RMSNORM_BWD_FIXED_MAX_DIM];

std::mutex g_setup_lock;
float* g_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch on the current device; looked up on first use.
cudaError_t scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> hold(g_setup_lock);
  if (g_scratch_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_dw_slices);
    if (e != cudaSuccess) return e;
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return cudaSuccess;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" int hb_rmsnorm_bwd_fixed_scratch(const void* dy, const void* h, const void* w,
                                            const float* rstd, const void* dres, void* dx, float* dw,
                                            int64_t rows, int64_t dim, float w_offset, void* stream) {
  if (dim <= 0 || dim % 8 != 0 || dim > HB_RMSNORM_BWD_FIXED_MAX_DIM || rows < 0 || rows > 0x7fffffffLL) {
    std::fputs("hb_rmsnorm_bwd_fixed_scratch: dim must be a multiple of 8 and at most 8192 "
               "(fixed 64 x 8192 float scratch), rows must fit in 31 bits\n", stderr);
    return HB_FIXED_ERR_SIZE;
  }
  if (!dy || !h || !w || !rstd || !dx || !dw || !aligned16(dy) || !aligned16(h) || !aligned16(w) ||
      !aligned16(dx) || (dres && !aligned16(dres))) {
    std::fputs("hb_rmsnorm_bwd_fixed_scratch: NULL or misaligned (16-byte) pointer\n", stderr);
    return HB_FIXED_ERR_POINTER;
  }
  float* slices = nullptr;
  cudaError_t e = scratch_for_current_device(&slices);
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    e = cudaMemsetAsync(dw, 0, sizeof(float) * dim, s);
    return static_cast<int>(e);
  }
  e = hb::rmsnorm_bwd(dy, h, w, rstd, dres, dx, slices, HB_RMSNORM_BWD_FIXED_SLICES,
                      static_cast<int>(rows), static_cast<int>(dim), w_offset, s);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = hb::colsum_f32(slices, HB_RMSNORM_BWD_FIXED_SLICES, static_cast<int>(dim), dw, false, false, s);
  return static_cast<int>(e);
}
