// Python bindings: thin torch-tensor front-ends over the raw-pointer launchers in this
// directory. No math happens here; every function checks its arguments, picks the
// current CUDA stream and calls one launcher.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "gemm.h"
#include "launch_count.h"
#include "ops.h"

namespace {

#define HB_CHECK_CUDA(x) TORCH_CHECK((x).is_cuda(), #x " must be a CUDA tensor")
#define HB_CHECK_BF16(x) TORCH_CHECK((x).scalar_type() == at::kBFloat16, #x " must be bfloat16")
#define HB_CUDA_OK(expr)                                                              \
  do {                                                                                \
    cudaError_t _e = (expr);                                                          \
    TORCH_CHECK(_e == cudaSuccess, "halite_b200 launch failed: ", cudaGetErrorString(_e)); \
    hb::launch_counter().fetch_add(1, std::memory_order_relaxed);                          \
  } while (0)

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int* status_ptr(const c10::optional<at::Tensor>& status) {
  if (!status.has_value()) return nullptr;
  TORCH_CHECK(status->is_cuda() && status->scalar_type() == at::kInt, "status must be cuda int32");
  return status->data_ptr<int>();
}

// out[M,N] (=|+=) op(a) * op(b). a: [M,K] (or [K,M] when a_mn), b: [N,K] (or [K,N] when b_mn).
// Optional fused gather description, filled from a Python dict (see hb::GatherParams).
bool fill_gather(const c10::optional<py::dict>& d, hb::GatherParams& gp) {
  if (!d.has_value()) return false;
  const py::dict& g = *d;
  auto srcs = g["src_ptrs"].cast<std::vector<int64_t>>();
  TORCH_CHECK((int)srcs.size() <= hb::kMaxPeers, "too many gather chunks");
  gp.n_chunks = (int)srcs.size();
  for (int i = 0; i < gp.n_chunks; ++i) gp.src[i] = reinterpret_cast<const void*>(srcs[i]);
  if (g.contains("peer_done_ptrs")) {
    auto pd = g["peer_done_ptrs"].cast<std::vector<int64_t>>();
    for (int i = 0; i < (int)pd.size() && i < hb::kMaxPeers; ++i) gp.peer_done[i] = reinterpret_cast<int*>(pd[i]);
  }
  gp.dst_base = reinterpret_cast<void*>(g["dst_ptr"].cast<int64_t>());
  gp.chunk_bytes = g["chunk_bytes"].cast<int64_t>();
  gp.granule_bytes = g["granule_bytes"].cast<int64_t>();
  gp.n_copy_ctas = g["n_copy_ctas"].cast<int>();
  gp.flags = reinterpret_cast<int*>(g["flags_ptr"].cast<int64_t>());
  gp.ready = g.contains("ready_ptr") ? reinterpret_cast<const int*>(g["ready_ptr"].cast<int64_t>()) : nullptr;
  gp.done_counter = g.contains("done_counter_ptr") ? reinterpret_cast<int*>(g["done_counter_ptr"].cast<int64_t>()) : nullptr;
  gp.epoch = g["epoch"].cast<int>();
  gp.dep = g["dep"].cast<int>();
  gp.dep_row_bytes = g["dep_row_bytes"].cast<int64_t>();
  gp.dep_base_offset = g.contains("dep_base_offset") ? g["dep_base_offset"].cast<int64_t>() : 0;
  gp.m_rot = g.contains("m_rot") ? g["m_rot"].cast<int>() : 0;
  gp.first_chunk = g.contains("first_chunk") ? g["first_chunk"].cast<int>() : 0;
  if (g.contains("reduce_out_ptr")) {
    gp.reduce_out = reinterpret_cast<float*>(g["reduce_out_ptr"].cast<int64_t>());
    gp.reduce_numel = g["reduce_numel"].cast<int64_t>();
    gp.reduce_scale = g["reduce_scale"].cast<float>();
    if (g.contains("mc_src_ptr")) gp.mc_src = reinterpret_cast<const float*>(g["mc_src_ptr"].cast<int64_t>());
  }
  return true;
}

bool fill_scatter(const c10::optional<py::dict>& d, hb::ScatterParams& sp) {
  if (!d.has_value()) return false;
  const py::dict& g = *d;
  auto dst = g["dst_ptrs"].cast<std::vector<int64_t>>();
  auto recv = g["recv_ptrs"].cast<std::vector<int64_t>>();
  auto pf = g["peer_flag_ptrs"].cast<std::vector<int64_t>>();
  TORCH_CHECK((int)dst.size() <= hb::kMaxPeers && dst.size() == recv.size() && dst.size() == pf.size(),
              "scatter pointer lists must have one entry per rank");
  sp.n_chunks = (int)dst.size();
  for (int i = 0; i < sp.n_chunks; ++i) {
    sp.dst[i] = reinterpret_cast<void*>(dst[i]);
    sp.recv[i] = reinterpret_cast<const void*>(recv[i]);
    sp.peer_flag[i] = reinterpret_cast<int*>(pf[i]);
  }
  sp.my_flags = reinterpret_cast<const int*>(g["my_flags_ptr"].cast<int64_t>());
  sp.out = reinterpret_cast<void*>(g["out_ptr"].cast<int64_t>());
  sp.cta_counter = reinterpret_cast<int*>(g["cta_counter_ptr"].cast<int64_t>());
  sp.rows_per_chunk = g["rows_per_chunk"].cast<int>();
  sp.rank = g["rank"].cast<int>();
  sp.epoch = g["epoch"].cast<int>();
  sp.m_rot = g.contains("m_rot") ? g["m_rot"].cast<int>() : 0;
  return true;
}

// Grouped (mixture-of-experts) description from a Python dict (see hb::GroupParams).
bool fill_group(const c10::optional<py::dict>& d, hb::GroupParams& gq) {
  if (!d.has_value()) return false;
  const py::dict& g = *d;
  gq.mode = g["mode"].cast<int>();
  if (gq.mode == 1) {
    gq.tile_group = reinterpret_cast<const int*>(g["tile_group_ptr"].cast<int64_t>());
    gq.b_group_rows = g["b_group_rows"].cast<int64_t>();
    gq.b_total_rows = g["b_total_rows"].cast<int64_t>();
  } else {
    gq.n_groups = g["n_groups"].cast<int>();
    gq.k_begin = reinterpret_cast<const int*>(g["k_begin_ptr"].cast<int64_t>());
    gq.k_end = reinterpret_cast<const int*>(g["k_end_ptr"].cast<int64_t>());
    gq.d_group_elems = g["d_group_elems"].cast<int64_t>();
  }
  return true;
}

void signal_flags(const std::vector<int64_t>& ptrs, int64_t epoch) {
  cudaError_t e = hb::signal_flags(ptrs.data(), (int)ptrs.size(), (int)epoch, cur_stream());
  TORCH_CHECK(e == cudaSuccess, "signal_flags failed: ", cudaGetErrorString(e));
  hb::launch_counter().fetch_add(1, std::memory_order_relaxed);
}

void wait_flags(const at::Tensor& flags, int64_t epoch, const c10::optional<at::Tensor>& status) {
  TORCH_CHECK(flags.is_cuda() && flags.scalar_type() == at::kInt && flags.is_contiguous());
  c10::cuda::CUDAGuard guard(flags.device());
  cudaError_t e = hb::wait_flags(flags.data_ptr<int>(), (int)flags.numel(), (int)epoch,
                                 status_ptr(status), cur_stream());
  TORCH_CHECK(e == cudaSuccess, "wait_flags failed: ", cudaGetErrorString(e));
  hb::launch_counter().fetch_add(1, std::memory_order_relaxed);
}

void gemm(const at::Tensor& a, const at::Tensor& b, at::Tensor& out, bool a_mn, bool b_mn,
          bool accumulate, int64_t block_n, int64_t max_ctas,
          const c10::optional<at::Tensor>& status, const c10::optional<py::dict>& gather,
          const c10::optional<py::dict>& scatter, const c10::optional<py::dict>& group) {
  HB_CHECK_CUDA(a); HB_CHECK_CUDA(b); HB_CHECK_CUDA(out);
  HB_CHECK_BF16(a); HB_CHECK_BF16(b);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && (out.dim() == 2 || group.has_value()), "gemm wants 2-D tensors");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && out.stride(-1) == 1,
              "gemm wants unit inner stride");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 || out.scalar_type() == at::kFloat,
              "gemm output must be bf16 or fp32");
  const int64_t M = a_mn ? a.size(1) : a.size(0);
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  int64_t N = b_mn ? b.size(1) : b.size(0);
  int64_t Kb = b_mn ? b.size(0) : b.size(1);
  hb::GroupParams gq;
  const bool grouped = fill_group(group, gq);
  if (grouped && gq.mode == 1) {
    // B stacks the groups along its rows: one group's share is the GEMM's N (K-major) or K (MN-major)
    if (b_mn) Kb = gq.b_group_rows; else N = gq.b_group_rows;
  }
  TORCH_CHECK(K == Kb, "gemm inner dimensions differ: ", K, " vs ", Kb);
  if (scatter.has_value()) {
    TORCH_CHECK(out.size(1) == N && out.is_contiguous(), "scatter mode wants a contiguous [rows, N] partial buffer");
  } else if (group.has_value()) {
    TORCH_CHECK(out.size(-1) == N && out.is_contiguous(), "grouped mode wants a contiguous output with N columns");
  } else {
    TORCH_CHECK(out.size(0) == M && out.size(1) == N, "gemm output shape mismatch");
  }
  c10::cuda::CUDAGuard guard(a.device());
  hb::GemmArgs g;
  g.a = a.data_ptr(); g.b = b.data_ptr(); g.d = out.data_ptr();
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.lda = (int)a.stride(0); g.ldb = (int)b.stride(0); g.ldd = (int)out.stride(-2);
  if (grouped) g.group = &gq;
  g.a_mn_major = a_mn; g.b_mn_major = b_mn;
  g.out_f32 = out.scalar_type() == at::kFloat;
  g.accumulate = accumulate;
  g.block_n = (int)block_n; g.max_ctas = (int)max_ctas;
  g.status = status_ptr(status);
  g.stream = cur_stream();
  hb::GatherParams gp;
  if (fill_gather(gather, gp)) g.gather = &gp;
  hb::ScatterParams sp;
  if (fill_scatter(scatter, sp)) g.scatter = &sp;
  cudaError_t err = hb::gemm_bf16(g);
  TORCH_CHECK(err == cudaSuccess, "halite_b200 gemm failed: ", cudaGetErrorString(err), " (M=", M,
              " N=", N, " K=", K, " lda=", g.lda, " ldb=", g.ldb, " ldd=", g.ldd, " a_mn=", a_mn,
              " b_mn=", b_mn, " out_f32=", g.out_f32, " a%16=", (uintptr_t)g.a % 16, " b%16=",
              (uintptr_t)g.b % 16, " d%16=", (uintptr_t)g.d % 16, ")");
  hb::launch_counter().fetch_add(1, std::memory_order_relaxed);
}

}  // namespace

void register_elementwise(pybind11::module_& m);  // ops_bindings.cpp
void register_infer(pybind11::module_& m);        // infer_bindings.cpp
void register_attention(pybind11::module_& m);    // attention_bindings.cpp

void register_runtime(py::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm, "bf16 tcgen05 GEMM", py::arg("a"), py::arg("b"), py::arg("out"),
        py::arg("a_mn") = false, py::arg("b_mn") = false, py::arg("accumulate") = false,
        py::arg("block_n") = 0, py::arg("max_ctas") = 0, py::arg("status") = py::none(),
        py::arg("gather") = py::none(), py::arg("scatter") = py::none(), py::arg("group") = py::none());
  m.def("gemm_set_peer_wait_sm_margin", [](int sms) { hb::gemm_set_peer_wait_sm_margin(sms); }, py::arg("sms"));
  m.def("gemm_peer_wait_sm_margin", []() { return hb::gemm_peer_wait_sm_margin(); });
  m.def("gemm_set_dynamic_schedule", [](bool on, bool force) { hb::gemm_set_dynamic_schedule(on, force); },
        "CTA-pair GEMM: hand work items out through a counter (true) or in fixed shares (false)",
        py::arg("on"), py::arg("force") = false);
  m.def("signal_flags", &signal_flags, "write epoch to flag words (possibly in peer memory)");
  m.def("wait_flags", &wait_flags, py::arg("flags"), py::arg("epoch"), py::arg("status") = py::none());
  m.def("launch_count", []() { return hb::launch_counter().load(); },
        "kernel launches issued through this extension so far");
  m.def("reset_launch_count", []() { hb::launch_counter().store(0); });
  register_elementwise(m);
  register_infer(m);
  register_attention(m);
  register_runtime(m);
}
