// Host entry points of the sm_100a GEMM family (no torch headers: raw pointers + stream).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hb {

struct GemmArgs {
  const void* a = nullptr;  // bf16
  const void* b = nullptr;  // bf16
  void* d = nullptr;        // bf16 or fp32, row-major [M, N]
  int M = 0, N = 0, K = 0;
  int lda = 0, ldb = 0, ldd = 0;  // leading dimensions in elements
  bool a_mn_major = false;        // false: A is [M, K] row-major; true: A is [K, M] row-major
  bool b_mn_major = false;        // false: B is [N, K] row-major; true: B is [K, N] row-major
  bool out_f32 = false;
  bool accumulate = false;  // D += A*B instead of D = A*B
  int block_n = 0;          // 0 = choose, else 128 or 256
  int max_ctas = 0;         // 0 = one per SM; >0 caps the grid (leaves SMs for a concurrent copy)
  int* status = nullptr;    // device int: set to a WaitCode when a bounded wait gave up
  cudaStream_t stream = nullptr;
};

cudaError_t gemm_bf16(const GemmArgs& args);
int gemm_pick_bn(int M, int N);

bool make_tmap_bf16_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                       uint64_t ld, uint32_t box_rows, uint32_t box_cols);

}  // namespace hb
