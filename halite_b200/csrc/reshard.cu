// Trainer -> rollout-engine weight hand-over in one launch: every destination tensor of the
// engine (a whole parameter, or this tensor-parallel rank's rows / columns of one, or its part of
// a packed q|k|v / gate|up matrix) is filled straight from the flat sharded parameter buffers of
// the data-parallel ranks. A source range may live in any rank's shard: the kernel resolves each
// 16-byte vector to (rank, offset) and reads it with a plain load through the peer mapping of
// that rank's buffer (NVLink), so no all-gather, no full tensor and no per-tensor collective is
// ever materialised.
//
// Replaces the per-tensor `full_tensor()` + copy loop of the reference
// (distributed/state_dict.py:5-38, infer/engine/model_runner.py:108-115).
#include <cuda_runtime.h>
#include <stdint.h>

#include "reshard.h"

namespace hb {

namespace {

__global__ void __launch_bounds__(256) reshard_kernel(const ReshardSegment* __restrict__ segs, int n_segs) {
  const ReshardSegment s = segs[blockIdx.y];
  const long vecs_per_row = s.row_bytes >> 4;
  const long total = static_cast<long>(s.rows) * vecs_per_row;
  uint4* __restrict__ dst = reinterpret_cast<uint4*>(s.dst);
  for (long v = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; v < total;
       v += static_cast<long>(gridDim.x) * blockDim.x) {
    const long row = v / vecs_per_row;
    const long flat = s.src_byte0 + row * s.src_pitch + ((v - row * vecs_per_row) << 4);
    const long rank = flat / s.shard_bytes;
    const long local = flat - rank * s.shard_bytes;
    dst[v] = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(s.src_base[rank]) + local);
  }
}

}  // namespace

cudaError_t reshard_copy(const ReshardSegment* segs_device, int n_segs, cudaStream_t stream) {
  if (n_segs <= 0) return cudaSuccess;
  dim3 grid(16, n_segs);
  reshard_kernel<<<grid, 256, 0, stream>>>(segs_device, n_segs);
  return cudaGetLastError();
}

}  // namespace hb
