// Raw-pointer launchers of the inference kernels (sm_100a). KV caches are
// [pages, 16, kv_heads, head_dim] bf16; page tables are [request slots, max_pages] int32.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace hb {

struct RopeAppendArgs {
  void* q = nullptr;            // [tokens, hq, dim] rotated in place (row stride q_stride)
  const void* k = nullptr;      // [tokens, hk, dim]
  const void* v = nullptr;
  void* k_cache = nullptr;
  void* v_cache = nullptr;
  const float* cos = nullptr;   // [max_pos, rot/2] or null (no rotation)
  const float* sin = nullptr;
  const int64_t* positions = nullptr;
  const int64_t* out_loc = nullptr;   // flat slot per token
  int tokens = 0, hq = 0, hk = 0, dim = 0, rot = 0;
  long q_stride = 0, k_stride = 0, v_stride = 0;
  bool interleaved = true;
  long cache_slots = 0;         // pages * 16, writes outside are dropped
};
cudaError_t rope_append(const RopeAppendArgs& a, cudaStream_t stream);

struct PagedDecodeArgs {
  const void* q = nullptr;      // [batch, hq, dim]
  const void* k_cache = nullptr;
  const void* v_cache = nullptr;
  void* out = nullptr;          // [batch, hq, dim] contiguous
  const int* page_table = nullptr;
  const int* req_slots = nullptr;
  const int* seq_lens = nullptr;
  float* workspace = nullptr;   // batch * hq * splits * (dim + 2) floats when splits > 1
  int batch = 0, hq = 0, hk = 0, dim = 0, max_pages = 0, splits = 1;
  long q_stride = 0, num_pages = 0;
  float scale = 1.f;
  int* status = nullptr;        // device int: set to 8 when a page id lies outside the pool
};
cudaError_t paged_decode(const PagedDecodeArgs& a, cudaStream_t stream);
int paged_decode_splits(int batch, int hk, int sm_count);

struct PagedPrefillArgs {
  const void* q = nullptr;      // [tokens, hq, dim] (row stride q_stride)
  const void* k_cache = nullptr;
  const void* v_cache = nullptr;
  void* out = nullptr;          // [tokens, hq, dim] (row stride o_stride)
  const int* page_table = nullptr;
  const int* req_slots = nullptr;
  const int* qo_indptr = nullptr;   // [batch + 1]
  const int* seq_lens = nullptr;    // [batch] keys per request (prefix + new)
  int batch = 0, hq = 0, hk = 0, dim = 0, max_pages = 0, max_extend = 0;
  long q_stride = 0, o_stride = 0, num_pages = 0;
  int* status = nullptr;            // device int: set to 8 when a page id lies outside the pool
  float scale = 1.f;
};
cudaError_t paged_prefill(const PagedPrefillArgs& a, cudaStream_t stream);

cudaError_t sample_gumbel(const float* logits, const float* temperature, const bool* greedy,
                          int64_t* ids, float* logprobs, int rows, int vocab, long ld, uint64_t seed,
                          uint64_t call, cudaStream_t stream);

}  // namespace hb
