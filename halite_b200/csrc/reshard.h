// One-launch copy from flat, rank-sharded parameter buffers into engine-layout tensors.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace hb {

constexpr int kReshardMaxRanks = 8;

// `rows` rows of `row_bytes` bytes each, written contiguously at `dst`. Row i starts at byte
// `src_byte0 + i * src_pitch` of a flat buffer that is cut into equal shards of `shard_bytes`
// bytes, shard r living at `src_base[r]` (this GPU's memory or a peer mapping). Every offset and
// length is a multiple of 16 bytes.
struct ReshardSegment {
  void* dst;
  const void* src_base[kReshardMaxRanks];
  long src_byte0;
  long src_pitch;
  long shard_bytes;
  long row_bytes;
  long rows;
};

cudaError_t reshard_copy(const ReshardSegment* segs_device, int n_segs, cudaStream_t stream);

}  // namespace hb
