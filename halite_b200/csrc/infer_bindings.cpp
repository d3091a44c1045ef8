// torch-tensor front-ends for the inference kernels declared in infer_kernels.h.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "infer_kernels.h"
#include "launch_count.h"

namespace {

#define HB_CUDA_OK(expr)                                                                   \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    TORCH_CHECK(_e == cudaSuccess, "halite_b200 launch failed: ", cudaGetErrorString(_e)); \
    hb::launch_counter().fetch_add(1, std::memory_order_relaxed);                          \
  } while (0)

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_cache(const at::Tensor& c, const char* name) {
  TORCH_CHECK(c.is_cuda() && c.scalar_type() == at::kBFloat16 && c.is_contiguous() && c.dim() == 4 &&
                  c.size(1) == 16,
              name, " must be a contiguous CUDA bf16 [pages, 16, kv_heads, head_dim] tensor");
}
void check_i32(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous(), name,
              " must be a contiguous CUDA int32 tensor");
}
void check_heads(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 3 && t.stride(2) == 1 &&
                  t.stride(1) == t.size(2),
              name, " must be CUDA bf16 [tokens, heads, head_dim] with packed heads");
}

// q (optional) rotated in place; k rotated into the cache; v copied into the cache.
void rope_append(const c10::optional<at::Tensor>& q, const at::Tensor& k, const at::Tensor& v,
                 at::Tensor& k_cache, at::Tensor& v_cache, const c10::optional<at::Tensor>& cos,
                 const c10::optional<at::Tensor>& sin, const c10::optional<at::Tensor>& positions,
                 const at::Tensor& out_loc, bool interleaved) {
  check_heads(k, "k");
  check_heads(v, "v");
  check_cache(k_cache, "k_cache");
  check_cache(v_cache, "v_cache");
  TORCH_CHECK(out_loc.is_cuda() && out_loc.scalar_type() == at::kLong && out_loc.is_contiguous());
  const int64_t T = k.size(0);
  TORCH_CHECK(out_loc.numel() == T && v.size(0) == T);
  TORCH_CHECK(k.size(1) == k_cache.size(2) && k.size(2) == k_cache.size(3), "k / cache shape mismatch");
  c10::cuda::CUDAGuard guard(k.device());
  hb::RopeAppendArgs a;
  if (q.has_value()) {
    check_heads(*q, "q");
    TORCH_CHECK(q->size(0) == T && q->size(2) == k.size(2));
    a.q = q->data_ptr();
    a.hq = (int)q->size(1);
    a.q_stride = q->stride(0);
  }
  a.k = k.data_ptr();
  a.v = v.data_ptr();
  a.k_cache = k_cache.data_ptr();
  a.v_cache = v_cache.data_ptr();
  a.dim = (int)k.size(2);
  a.rot = a.dim;
  if (cos.has_value()) {
    TORCH_CHECK(sin.has_value() && positions.has_value(), "cos needs sin and positions");
    TORCH_CHECK(cos->is_cuda() && cos->scalar_type() == at::kFloat && cos->is_contiguous());
    TORCH_CHECK(sin->is_cuda() && sin->scalar_type() == at::kFloat && sin->is_contiguous());
    TORCH_CHECK(positions->is_cuda() && positions->scalar_type() == at::kLong &&
                positions->is_contiguous() && positions->numel() == T);
    a.cos = cos->data_ptr<float>();
    a.sin = sin->data_ptr<float>();
    a.positions = positions->data_ptr<int64_t>();
    a.rot = (int)cos->size(-1) * 2;
  }
  a.out_loc = out_loc.data_ptr<int64_t>();
  a.tokens = (int)T;
  a.hk = (int)k.size(1);
  a.k_stride = k.stride(0);
  a.v_stride = v.stride(0);
  a.interleaved = interleaved;
  a.cache_slots = k_cache.size(0) * 16;
  HB_CUDA_OK(hb::rope_append(a, cur_stream()));
}

void kv_append(at::Tensor& k_cache, at::Tensor& v_cache, const at::Tensor& k, const at::Tensor& v,
               const at::Tensor& out_loc) {
  rope_append(c10::nullopt, k, v, k_cache, v_cache, c10::nullopt, c10::nullopt, c10::nullopt, out_loc,
              true);
}

void paged_decode(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache,
                  at::Tensor& out, const at::Tensor& page_table, const at::Tensor& req_slots,
                  const at::Tensor& seq_lens, const c10::optional<at::Tensor>& workspace, double scale,
                  const c10::optional<at::Tensor>& status) {
  check_heads(q, "q");
  check_cache(k_cache, "k_cache");
  check_cache(v_cache, "v_cache");
  check_i32(page_table, "page_table");
  check_i32(req_slots, "req_slots");
  check_i32(seq_lens, "seq_lens");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.is_contiguous() &&
              out.numel() == q.size(0) * q.size(1) * q.size(2));
  c10::cuda::CUDAGuard guard(q.device());
  hb::PagedDecodeArgs a;
  a.q = q.data_ptr();
  a.k_cache = k_cache.data_ptr();
  a.v_cache = v_cache.data_ptr();
  a.out = out.data_ptr();
  a.page_table = page_table.data_ptr<int>();
  a.req_slots = req_slots.data_ptr<int>();
  a.seq_lens = seq_lens.data_ptr<int>();
  a.batch = (int)q.size(0);
  a.hq = (int)q.size(1);
  a.hk = (int)k_cache.size(2);
  a.dim = (int)q.size(2);
  a.max_pages = (int)page_table.size(1);
  a.q_stride = q.stride(0);
  a.num_pages = k_cache.size(0);
  a.scale = (float)scale;
  if (status.has_value()) a.status = status->data_ptr<int>();
  a.splits = hb::paged_decode_splits(a.batch, a.hk,
                                     at::cuda::getCurrentDeviceProperties()->multiProcessorCount);
  if (a.splits > 1) {
    const int64_t need = (int64_t)a.batch * a.hq * a.splits * (a.dim + 2);
    if (workspace.has_value() && workspace->numel() >= need) {
      TORCH_CHECK(workspace->is_cuda() && workspace->scalar_type() == at::kFloat);
      a.workspace = workspace->data_ptr<float>();
    } else {
      // without a large enough caller workspace fall back to fewer splits that fit, or one
      int64_t have = workspace.has_value() ? workspace->numel() : 0;
      int s = (int)(have / ((int64_t)a.batch * a.hq * (a.dim + 2)));
      if (s >= 2) {
        a.splits = s;
        a.workspace = workspace->data_ptr<float>();
      } else {
        a.splits = 1;
      }
    }
  }
  HB_CUDA_OK(hb::paged_decode(a, cur_stream()));
}

void paged_prefill(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache,
                   at::Tensor& out, const at::Tensor& page_table, const at::Tensor& req_slots,
                   const at::Tensor& qo_indptr, const at::Tensor& seq_lens, int64_t max_extend,
                   double scale, const c10::optional<at::Tensor>& status) {
  check_heads(q, "q");
  check_heads(out, "out");
  check_cache(k_cache, "k_cache");
  check_cache(v_cache, "v_cache");
  check_i32(page_table, "page_table");
  check_i32(req_slots, "req_slots");
  check_i32(qo_indptr, "qo_indptr");
  check_i32(seq_lens, "seq_lens");
  TORCH_CHECK(out.sizes() == q.sizes());
  c10::cuda::CUDAGuard guard(q.device());
  hb::PagedPrefillArgs a;
  a.q = q.data_ptr();
  a.k_cache = k_cache.data_ptr();
  a.v_cache = v_cache.data_ptr();
  a.out = out.data_ptr();
  a.page_table = page_table.data_ptr<int>();
  a.req_slots = req_slots.data_ptr<int>();
  a.qo_indptr = qo_indptr.data_ptr<int>();
  a.seq_lens = seq_lens.data_ptr<int>();
  a.batch = (int)req_slots.numel();
  a.hq = (int)q.size(1);
  a.hk = (int)k_cache.size(2);
  a.dim = (int)q.size(2);
  a.max_pages = (int)page_table.size(1);
  a.max_extend = (int)max_extend;
  a.q_stride = q.stride(0);
  a.o_stride = out.stride(0);
  a.num_pages = k_cache.size(0);
  a.scale = (float)scale;
  if (status.has_value()) a.status = status->data_ptr<int>();
  HB_CUDA_OK(hb::paged_prefill(a, cur_stream()));
}

std::tuple<at::Tensor, at::Tensor> sample_gumbel(const at::Tensor& logits, const at::Tensor& temperature,
                                                 const at::Tensor& greedy, int64_t seed, int64_t call) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 &&
              logits.stride(1) == 1);
  TORCH_CHECK(temperature.is_cuda() && temperature.scalar_type() == at::kFloat &&
              temperature.is_contiguous() && temperature.numel() == logits.size(0));
  TORCH_CHECK(greedy.is_cuda() && greedy.scalar_type() == at::kBool && greedy.is_contiguous() &&
              greedy.numel() == logits.size(0));
  c10::cuda::CUDAGuard guard(logits.device());
  at::Tensor ids = at::empty({logits.size(0)}, logits.options().dtype(at::kLong));
  at::Tensor lp = at::empty({logits.size(0)}, logits.options());
  HB_CUDA_OK(hb::sample_gumbel(logits.data_ptr<float>(), temperature.data_ptr<float>(),
                               greedy.data_ptr<bool>(), ids.data_ptr<int64_t>(), lp.data_ptr<float>(),
                               (int)logits.size(0), (int)logits.size(1), logits.stride(0),
                               (uint64_t)seed, (uint64_t)call, cur_stream()));
  return {ids, lp};
}

}  // namespace

void register_infer(pybind11::module_& m) {
  namespace py = pybind11;
  m.def("rope_append", &rope_append, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("k_cache"),
        py::arg("v_cache"), py::arg("cos"), py::arg("sin"), py::arg("positions"), py::arg("out_loc"),
        py::arg("interleaved") = true);
  m.def("kv_append", &kv_append);
  m.def("paged_decode", &paged_decode, py::arg("q"), py::arg("k_cache"), py::arg("v_cache"),
        py::arg("out"), py::arg("page_table"), py::arg("req_slots"), py::arg("seq_lens"),
        py::arg("workspace"), py::arg("scale"), py::arg("status") = py::none());
  m.def("paged_prefill", &paged_prefill, py::arg("q"), py::arg("k_cache"), py::arg("v_cache"), py::arg("out"),
        py::arg("page_table"), py::arg("req_slots"), py::arg("qo_indptr"), py::arg("seq_lens"), py::arg("max_extend"),
        py::arg("scale"), py::arg("status") = py::none());
  m.def("sample_gumbel", &sample_gumbel);
}
