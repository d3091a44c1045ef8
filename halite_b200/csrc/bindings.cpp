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
void gemm(const at::Tensor& a, const at::Tensor& b, at::Tensor& out, bool a_mn, bool b_mn,
          bool accumulate, int64_t block_n, int64_t max_ctas,
          const c10::optional<at::Tensor>& status) {
  HB_CHECK_CUDA(a); HB_CHECK_CUDA(b); HB_CHECK_CUDA(out);
  HB_CHECK_BF16(a); HB_CHECK_BF16(b);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2, "gemm wants 2-D tensors");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1,
              "gemm wants unit inner stride");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 || out.scalar_type() == at::kFloat,
              "gemm output must be bf16 or fp32");
  const int64_t M = a_mn ? a.size(1) : a.size(0);
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  const int64_t Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm inner dimensions differ: ", K, " vs ", Kb);
  TORCH_CHECK(out.size(0) == M && out.size(1) == N, "gemm output shape mismatch");
  c10::cuda::CUDAGuard guard(a.device());
  hb::GemmArgs g;
  g.a = a.data_ptr(); g.b = b.data_ptr(); g.d = out.data_ptr();
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.lda = (int)a.stride(0); g.ldb = (int)b.stride(0); g.ldd = (int)out.stride(0);
  g.a_mn_major = a_mn; g.b_mn_major = b_mn;
  g.out_f32 = out.scalar_type() == at::kFloat;
  g.accumulate = accumulate;
  g.block_n = (int)block_n; g.max_ctas = (int)max_ctas;
  g.status = status_ptr(status);
  g.stream = cur_stream();
  cudaError_t err = hb::gemm_bf16(g);
  TORCH_CHECK(err == cudaSuccess, "halite_b200 gemm failed: ", cudaGetErrorString(err), " (M=", M,
              " N=", N, " K=", K, " lda=", g.lda, " ldb=", g.ldb, " ldd=", g.ldd, " a_mn=", a_mn,
              " b_mn=", b_mn, " out_f32=", g.out_f32, " a%16=", (uintptr_t)g.a % 16, " b%16=",
              (uintptr_t)g.b % 16, " d%16=", (uintptr_t)g.d % 16, ")");
  hb::launch_counter().fetch_add(1, std::memory_order_relaxed);
}

}  // namespace

void register_elementwise(pybind11::module_& m);  // ops_bindings.cpp

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm, "bf16 tcgen05 GEMM", py::arg("a"), py::arg("b"), py::arg("out"),
        py::arg("a_mn") = false, py::arg("b_mn") = false, py::arg("accumulate") = false,
        py::arg("block_n") = 0, py::arg("max_ctas") = 0, py::arg("status") = py::none());
  m.def("launch_count", []() { return hb::launch_counter().load(); },
        "kernel launches issued through this extension so far");
  m.def("reset_launch_count", []() { hb::launch_counter().store(0); });
  register_elementwise(m);
}
