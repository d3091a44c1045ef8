// Host entry points of the sm_100a GEMM family (no torch headers: raw pointers + stream).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hb {

constexpr int kMaxPeers = 8;
constexpr int kClusterSplitBlockN = 1064;   // GemmArgs::block_n value that forces the cluster split-K kernel (64-column tiles)
constexpr int kPairBlockN = 512;   // GemmArgs::block_n value that forces the CTA-pair (cta_group::2) kernel

// Side job that a GEMM launch can carry: a few CTAs copy `n_chunks` equal chunks (each from a
// peer GPU's memory, or from local memory) into one contiguous local destination while the
// remaining CTAs compute; a tile whose operand rows lie in the destination waits only for the
// granules it reads. This is how an all-gather is fused into the GEMM that consumes it:
//   dep = 1: the A operand (M rows) is the gathered buffer  (TP all-gather -> GEMM)
//   dep = 2: the B operand (N rows) lies inside the gathered buffer (FSDP parameter all-gather
//            fused into the first GEMM that uses the unit's parameters)
// Remote data is pulled with plain loads into local memory and fed to the tensor cores by TMA
// from there; no TMA load ever names remote memory.
struct GatherParams {
  const void* src[kMaxPeers] = {};   // chunk i comes from src[i]; nullptr = already in place
  int* peer_done[kMaxPeers] = {};    // written with `epoch` (system scope) once chunk i was read
  void* dst_base = nullptr;          // chunk i lands at dst_base + i * chunk_bytes
  long chunk_bytes = 0;
  long granule_bytes = 0;            // flag granularity (multiple of 16)
  int n_chunks = 0;
  int n_copy_ctas = 0;
  int* flags = nullptr;              // [n_chunks * granules_per_chunk] local; set to `epoch`
  const int* ready = nullptr;        // [n_chunks] local; chunk i may be read once ready[i] >= epoch
  int* done_counter = nullptr;       // local scratch counter (zeroed by the launcher)
  int epoch = 1;
  int dep = 0;
  long dep_row_bytes = 0;            // bytes between consecutive operand rows in the destination
  long dep_base_offset = 0;          // byte offset of operand row 0 inside the destination
  int m_rot = 0;                     // first M tile to compute (start on the local chunk)
  int first_chunk = 0;               // chunk handled first by the copy CTAs (the local one)
  // Reduce mode (reduce_out != nullptr): instead of copying, the copy CTAs compute
  //   reduce_out[i] = reduce_scale * sum over chunks c of ((const float*)src[c])[i],  i < reduce_numel
  // in chunk order (the same order on every rank), i.e. this rank's part of a reduce-scatter of
  // fp32 buffers that live in every rank's memory; src[c] is chunk c's buffer already offset to
  // this rank's range (own buffer included). `ready` / `peer_done` work as above.
  float* reduce_out = nullptr;
  long reduce_numel = 0;
  float reduce_scale = 1.f;
  // Reduce mode through the switch: when the buffers are bound to an NVLink multicast object,
  // `mc_src` is the multicast address of this rank's range; one `multimem.ld_reduce` per 16 bytes
  // then returns the sum over all ranks (added inside NVSwitch) instead of one load per rank.
  const float* mc_src = nullptr;
};

// Fused GEMM -> reduce-scatter over the M dimension. Output rows are split into `n_chunks`
// equal chunks, chunk c belonging to rank c. The epilogue stores each tile straight to its
// owner: the local partial buffer for the own chunk, the owner's receive slot (peer memory)
// for the others. When all tiles are out, the CTAs tell every peer (one flag each), wait for
// the peers' flags and sum own partial + received partials into `out` (bf16), all in the same
// launch. `dst` / `recv` buffers are bf16 [rows_per_chunk, N] with leading dimension N.
struct ScatterParams {
  void* dst[kMaxPeers] = {};        // where this rank's partial of chunk c goes (peer memory for c != rank)
  const void* recv[kMaxPeers] = {}; // local slots holding rank p's partial of this rank's chunk (nullptr for p == rank)
  int* peer_flag[kMaxPeers] = {};   // flag word on rank p that announces "my partials for you are written"
  const int* my_flags = nullptr;    // local flag words, one per peer, written by the peers
  void* out = nullptr;              // [rows_per_chunk, N] bf16 reduced result
  int* cta_counter = nullptr;       // local scratch (zeroed by the launcher)
  int rows_per_chunk = 0;
  int n_chunks = 0;                 // 0 = scatter disabled
  int rank = 0;
  int epoch = 1;
  int m_rot = 0;                    // first M tile to compute (start on a peer's rows so they travel early)
};

// Grouped GEMM (mixture-of-experts layers): one launch covers every expert, with the tile table on
// the device so the host never needs the per-expert token counts.
//   mode 1 (forward, dgrad): A / D rows are laid out expert by expert, every expert's block padded
//     to a multiple of 128 rows, so each 128-row tile belongs to one expert: `tile_group[tile]`
//     (-1: no expert, the tile is skipped). B stacks the experts' matrices along its row
//     dimension (`b_group_rows` rows each, `b_total_rows` in all).
//   mode 2 (wgrad): D[e] = A[rows of e]^T B[rows of e] for every expert e; the K range of expert e is
//     rows [k_begin[e], k_end[e]) (multiples of 64, padding rows are zero), outputs are
//     `d_group_elems` apart. GemmArgs::K is the total number of rows.
struct GroupParams {
  int mode = 0;
  const int* tile_group = nullptr;
  long b_group_rows = 0;
  long b_total_rows = 0;
  int n_groups = 0;
  const int* k_begin = nullptr;
  const int* k_end = nullptr;
  long d_group_elems = 0;
};

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
  int block_n = 0;          // 0 = choose, else 64, 128 or 256 (one CTA per tile) or kPairBlockN
  int max_ctas = 0;         // 0 = one per SM; >0 caps the grid (leaves SMs for a concurrent copy)
  int* status = nullptr;    // device int: set to a WaitCode when a bounded wait gave up
  const GatherParams* gather = nullptr;  // optional fused gather (see above)
  const ScatterParams* scatter = nullptr;  // optional fused reduce-scatter (bf16 output only)
  const GroupParams* group = nullptr;      // optional grouped mode (single-CTA kernel, no split / collectives)
  cudaStream_t stream = nullptr;
};

cudaError_t gemm_bf16(const GemmArgs& args);
cudaError_t signal_flags(const int64_t* ptrs, int n, int epoch, cudaStream_t stream);
cudaError_t wait_flags(const int* flags, int n, int epoch, int* status, cudaStream_t stream);
int gemm_pick_bn(int M, int N);
// Pair kernel: hand work items out through a counter, or in fixed shares (default). A setting from
// the environment (HB_GEMM_DYNAMIC=0/1) wins unless `force`.
void gemm_set_dynamic_schedule(bool on, bool force = false);
// SMs left free by GEMM launches whose CTAs spin on a peer GPU's progress (tile-dependent gather, scatter),
// so that a collective of another process group running beside them always finds room. 0 = none.
void gemm_set_peer_wait_sm_margin(int sms);
int gemm_peer_wait_sm_margin();

bool make_tmap_bf16_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                       uint64_t ld, uint32_t box_rows, uint32_t box_cols);

}  // namespace hb
