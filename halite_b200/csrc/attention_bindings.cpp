// torch-tensor front-ends for the training attention kernels declared in attention.h.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "attention.h"
#include "launch_count.h"
#include "reshard.h"

namespace {

#define HB_ATTN_OK(expr, n)                                                                   \
  do {                                                                                        \
    cudaError_t _e = (expr);                                                                  \
    TORCH_CHECK(_e == cudaSuccess, "halite_b200 attention launch failed: ", cudaGetErrorString(_e)); \
    hb::launch_counter().fetch_add((n), std::memory_order_relaxed);                           \
  } while (0)

// x: [..., heads, head_dim] bf16 view whose leading dims collapse to one token stride
int64_t token_stride(const at::Tensor& x, const char* name) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16, name, " must be a CUDA bf16 tensor");
  const int64_t d = x.size(-1);
  TORCH_CHECK(x.dim() >= 3 && x.stride(-1) == 1 && x.stride(-2) == d, name, ": heads must be adjacent");
  for (int i = x.dim() - 4; i >= 0; --i)
    TORCH_CHECK(x.size(i) == 1 || x.stride(i) == x.stride(i + 1) * x.size(i + 1), name,
                ": token dims must be collapsible");
  return x.stride(-3);
}

hb::AttnArgs make_args(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                       const c10::optional<at::Tensor>& seg_start, const c10::optional<at::Tensor>& seg_end,
                       int64_t seq_len, bool causal, int64_t window, double scale, double softcap,
                       const c10::optional<at::Tensor>& status) {
  hb::AttnArgs a;
  a.q = q.data_ptr();
  a.k = k.data_ptr();
  a.v = v.data_ptr();
  a.q_tok_stride = token_stride(q, "q");
  a.k_tok_stride = token_stride(k, "k");
  a.v_tok_stride = token_stride(v, "v");
  a.head_dim = (int)q.size(-1);
  a.n_heads = (int)q.size(-2);
  a.n_kv_heads = (int)k.size(-2);
  const int64_t total = q.numel() / (q.size(-1) * q.size(-2));
  TORCH_CHECK(total < (1LL << 31), "too many tokens");
  TORCH_CHECK(k.numel() / (k.size(-1) * k.size(-2)) == total && v.sizes() == k.sizes() && k.size(-1) == q.size(-1),
              "q, k, v must cover the same tokens (self-attention) with one head_dim");
  a.total = (int)total;
  a.seq_len = (int)seq_len;
  if (seg_start.has_value()) {
    TORCH_CHECK(seg_end.has_value(), "seg_start needs seg_end");
    for (const at::Tensor* t : {&*seg_start, &*seg_end})
      TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->is_contiguous() && t->numel() == total,
                  "segment bounds must be contiguous CUDA int32, one per token");
    a.seg_start = seg_start->data_ptr<int>();
    a.seg_end = seg_end->data_ptr<int>();
  }
  a.causal = causal;
  a.window = (int)window;
  a.scale = (float)scale;
  a.softcap = (float)softcap;
  if (status.has_value()) a.status = status->data_ptr<int>();
  a.stream = at::cuda::getCurrentCUDAStream().stream();
  return a;
}

// returns (out [same leading dims as q, heads, head_dim] contiguous, lse fp32 [heads, total])
std::tuple<at::Tensor, at::Tensor> attention_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                                 const c10::optional<at::Tensor>& seg_start,
                                                 const c10::optional<at::Tensor>& seg_end, int64_t seq_len,
                                                 bool causal, int64_t window, double scale, double softcap,
                                                 const c10::optional<at::Tensor>& status) {
  c10::cuda::CUDAGuard guard(q.device());
  hb::AttnArgs a = make_args(q, k, v, seg_start, seg_end, seq_len, causal, window, scale, softcap, status);
  at::Tensor out = at::empty(q.sizes(), q.options());
  at::Tensor lse = at::empty({(int64_t)a.n_heads, (int64_t)a.total}, q.options().dtype(at::kFloat));
  HB_ATTN_OK(hb::attention_fwd(a, out.data_ptr(), lse.data_ptr<float>()), 1);
  return {out, lse};
}

// dq / dk / dv are written into the given views (slots of a packed gradient are fine). With
// cos / sin / positions, dq is rotated back on its way out (inverse RoPE).
void attention_bwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& out,
                   const at::Tensor& d_out, const at::Tensor& lse, at::Tensor& dq, at::Tensor& dk, at::Tensor& dv,
                   const c10::optional<at::Tensor>& seg_start, const c10::optional<at::Tensor>& seg_end,
                   int64_t seq_len, bool causal, int64_t window, double scale, double softcap,
                   const c10::optional<at::Tensor>& status, const c10::optional<at::Tensor>& cos,
                   const c10::optional<at::Tensor>& sin, const c10::optional<at::Tensor>& positions, int64_t rot_dim,
                   bool interleaved) {
  c10::cuda::CUDAGuard guard(q.device());
  hb::AttnArgs a = make_args(q, k, v, seg_start, seg_end, seq_len, causal, window, scale, softcap, status);
  TORCH_CHECK(out.is_contiguous() && d_out.is_contiguous() && out.scalar_type() == at::kBFloat16 &&
                  d_out.scalar_type() == at::kBFloat16 && out.numel() == q.numel() && d_out.numel() == q.numel(),
              "out / d_out must be contiguous bf16 shaped like q");
  TORCH_CHECK(lse.is_contiguous() && lse.scalar_type() == at::kFloat && lse.numel() == (int64_t)a.n_heads * a.total,
              "lse must be fp32 [heads, tokens]");
  TORCH_CHECK(dq.sizes() == q.sizes() && dk.sizes() == k.sizes() && dv.sizes() == v.sizes(),
              "dq / dk / dv must be shaped like q / k / v");
  const int64_t dqs = token_stride(dq, "dq"), dks = token_stride(dk, "dk"), dvs = token_stride(dv, "dv");
  hb::AttnDqRotation rot;
  if (cos.has_value() && rot_dim > 0) {
    TORCH_CHECK(sin.has_value() && positions.has_value(), "rotation needs cos, sin and positions");
    TORCH_CHECK(cos->is_cuda() && cos->scalar_type() == at::kFloat && cos->is_contiguous() &&
                    sin->scalar_type() == at::kFloat && sin->is_contiguous() && cos->size(-1) * 2 == rot_dim,
                "cos / sin must be contiguous fp32 [max_position, rot_dim / 2]");
    TORCH_CHECK(positions->is_cuda() && positions->is_contiguous() && positions->numel() == a.total &&
                    (positions->scalar_type() == at::kLong || positions->scalar_type() == at::kInt),
                "positions must be contiguous CUDA int32 / int64, one per token");
    rot.cos = cos->data_ptr<float>();
    rot.sin = sin->data_ptr<float>();
    rot.positions = positions->data_ptr();
    rot.pos_is_i64 = positions->scalar_type() == at::kLong;
    rot.rot_dim = (int)rot_dim;
    rot.interleaved = interleaved;
  }
  at::Tensor delta = at::empty_like(lse);
  at::Tensor dq_accum = at::empty(q.sizes(), q.options().dtype(at::kFloat));
  HB_ATTN_OK(hb::attention_bwd(a, out.data_ptr(), d_out.data_ptr(), lse.data_ptr<float>(), delta.data_ptr<float>(),
                               dq_accum.data_ptr<float>(), dq.data_ptr(), dqs, rot, dk.data_ptr(), dks, dv.data_ptr(),
                               dvs),
             3);
}

// `table`: int64 [n, 14] on the device, rows laid out as hb::ReshardSegment
// (dst, src_base[8], src_byte0, src_pitch, shard_bytes, row_bytes, rows).
void reshard_copy(const at::Tensor& table) {
  static_assert(sizeof(hb::ReshardSegment) == 14 * sizeof(int64_t), "segment layout");
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kLong && table.is_contiguous() && table.dim() == 2 &&
                  table.size(1) == 14, "segment table must be a contiguous CUDA int64 [n, 14] tensor");
  c10::cuda::CUDAGuard guard(table.device());
  HB_ATTN_OK(hb::reshard_copy(reinterpret_cast<const hb::ReshardSegment*>(table.data_ptr<int64_t>()),
                              (int)table.size(0), at::cuda::getCurrentCUDAStream().stream()),
             1);
}

}  // namespace

void register_attention(pybind11::module_& m) {
  namespace py = pybind11;
  m.def("attention_fwd", &attention_fwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("seg_start") = py::none(),
        py::arg("seg_end") = py::none(), py::arg("seq_len") = 0, py::arg("causal") = true, py::arg("window") = 0,
        py::arg("scale") = 1.0, py::arg("softcap") = 0.0, py::arg("status") = py::none());
  m.def("reshard_copy", &reshard_copy, py::arg("table"));
#ifdef HB_ATTN_PROFILE
  m.def("attention_profile_read", [](bool reset) {
    unsigned long long v[32];
    HB_ATTN_OK(hb::attention_profile_read(v, reset), 1);
    return std::vector<unsigned long long>(v, v + 32);
  }, py::arg("reset") = true);
#endif
  m.def("attention_bwd", &attention_bwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("out"), py::arg("d_out"),
        py::arg("lse"), py::arg("dq"), py::arg("dk"), py::arg("dv"), py::arg("seg_start") = py::none(),
        py::arg("seg_end") = py::none(), py::arg("seq_len") = 0, py::arg("causal") = true, py::arg("window") = 0,
        py::arg("scale") = 1.0, py::arg("softcap") = 0.0, py::arg("status") = py::none(),
        py::arg("cos") = py::none(), py::arg("sin") = py::none(), py::arg("positions") = py::none(),
        py::arg("rot_dim") = 0, py::arg("interleaved") = true);
}
