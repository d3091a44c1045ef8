// torch-tensor front-ends for the launchers declared in ops.h.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "launch_count.h"
#include "ops.h"

namespace {

#define HB_CUDA_OK(expr)                                                                   \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    TORCH_CHECK(_e == cudaSuccess, "halite_b200 launch failed: ", cudaGetErrorString(_e)); \
    hb::launch_counter().fetch_add(1, std::memory_order_relaxed);                          \
  } while (0)

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_bf16(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous(), name,
              " must be a contiguous CUDA bf16 tensor");
}
void check_f32(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous(), name,
              " must be a contiguous CUDA fp32 tensor");
}
const void* opt_ptr(const c10::optional<at::Tensor>& t) {
  return t.has_value() ? t->data_ptr() : nullptr;
}

// returns (y, h_out or None, rstd)
std::tuple<at::Tensor, c10::optional<at::Tensor>, at::Tensor> rmsnorm_fwd(
    const at::Tensor& x, const c10::optional<at::Tensor>& residual, const at::Tensor& w, double eps,
    double w_offset, bool write_h) {
  check_bf16(x, "x");
  check_bf16(w, "w");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t dim = x.size(-1);
  const int64_t rows = x.numel() / dim;
  if (residual.has_value()) check_bf16(*residual, "residual");
  at::Tensor y = at::empty_like(x);
  at::Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  c10::optional<at::Tensor> h;
  if (residual.has_value() && write_h) h = at::empty_like(x);
  HB_CUDA_OK(hb::rmsnorm_fwd(x.data_ptr(), opt_ptr(residual), w.data_ptr(), y.data_ptr(),
                             h.has_value() ? h->data_ptr() : nullptr, rstd.data_ptr<float>(),
                             (int)rows, (int)dim, (float)eps, (float)w_offset, cur_stream()));
  return {y, h, rstd};
}

// returns (dx, dw fp32)
std::tuple<at::Tensor, at::Tensor> rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& h,
                                               const at::Tensor& w, const at::Tensor& rstd,
                                               const c10::optional<at::Tensor>& dres,
                                               double w_offset) {
  check_bf16(dy, "dy");
  check_bf16(h, "h");
  check_bf16(w, "w");
  check_f32(rstd, "rstd");
  c10::cuda::CUDAGuard guard(dy.device());
  const int64_t dim = h.size(-1);
  const int64_t rows = h.numel() / dim;
  if (dres.has_value()) check_bf16(*dres, "dres");
  at::Tensor dx = at::empty_like(h);
  const int prows = at::cuda::getCurrentDeviceProperties()->multiProcessorCount * 2;
  at::Tensor partial = at::empty({prows, dim}, h.options().dtype(at::kFloat));
  at::Tensor dw = at::empty({dim}, h.options().dtype(at::kFloat));
  HB_CUDA_OK(hb::rmsnorm_bwd(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(),
                             opt_ptr(dres), dx.data_ptr(), partial.data_ptr<float>(), prows,
                             (int)rows, (int)dim, (float)w_offset, cur_stream()));
  HB_CUDA_OK(hb::colsum_f32(partial.data_ptr<float>(), prows, (int)dim, dw.data_ptr(), false, false,
                            cur_stream()));
  return {dx, dw};
}

// x: [..., heads, head_dim] view whose token stride may exceed heads*head_dim (slices of a
// fused qkv output); rotated in place.
void rope_(at::Tensor& x, const at::Tensor& cos, const at::Tensor& sin, const at::Tensor& positions,
           int64_t rot_dim, bool interleaved, bool conjugate) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16, "x must be CUDA bf16");
  TORCH_CHECK(x.dim() >= 3, "x must be [..., heads, head_dim]");
  check_f32(cos, "cos");
  check_f32(sin, "sin");
  TORCH_CHECK(positions.is_cuda() && positions.is_contiguous() &&
                  (positions.scalar_type() == at::kLong || positions.scalar_type() == at::kInt),
              "positions must be contiguous CUDA int32/int64");
  const int64_t head_dim = x.size(-1), heads = x.size(-2);
  TORCH_CHECK(x.stride(-1) == 1 && x.stride(-2) == head_dim, "heads must be packed");
  const int64_t tokens = x.numel() / (heads * head_dim);
  TORCH_CHECK(positions.numel() == tokens, "one position per token");
  // leading dims must be collapsible to one token dim with a single stride
  int64_t token_stride = x.stride(-3);
  for (int d = x.dim() - 4; d >= 0; --d)
    TORCH_CHECK(x.size(d) == 1 || x.stride(d) == x.stride(d + 1) * x.size(d + 1),
                "token dims of x must be collapsible");
  TORCH_CHECK(cos.size(-1) * 2 == rot_dim, "cos/sin tables must be [max_pos, rot_dim/2]");
  c10::cuda::CUDAGuard guard(x.device());
  HB_CUDA_OK(hb::rope_inplace(x.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(),
                              positions.data_ptr(), positions.scalar_type() == at::kLong,
                              (int)tokens, (int)heads, (int)head_dim, (int)rot_dim, token_stride,
                              interleaved, conjugate, cur_stream()));
}

static int64_t collapsed_token_stride(const at::Tensor& x, const char* name) {
  const int64_t head_dim = x.size(-1);
  TORCH_CHECK(x.dim() >= 3 && x.stride(-1) == 1 && x.stride(-2) == head_dim, name, ": heads must be packed");
  for (int d = x.dim() - 4; d >= 0; --d)
    TORCH_CHECK(x.size(d) == 1 || x.stride(d) == x.stride(d + 1) * x.size(d + 1), name,
                ": token dims must be collapsible");
  return x.stride(-3);
}

// dst[..., heads, head_dim] = rotate(src[..., heads, head_dim]); both may be strided views (slices
// of packed qkv tensors). Without tables (rot_dim = 0) this is a strided copy.
void rope_copy(const at::Tensor& src, at::Tensor& dst, const c10::optional<at::Tensor>& cos,
               const c10::optional<at::Tensor>& sin, const c10::optional<at::Tensor>& positions, int64_t rot_dim,
               bool interleaved, bool conjugate) {
  TORCH_CHECK(src.is_cuda() && src.scalar_type() == at::kBFloat16 && dst.is_cuda() &&
                  dst.scalar_type() == at::kBFloat16, "src/dst must be CUDA bf16");
  TORCH_CHECK(src.sizes() == dst.sizes(), "src/dst shapes differ");
  const int64_t head_dim = src.size(-1), heads = src.size(-2);
  const int64_t tokens = src.numel() / (heads * head_dim);
  const int64_t ss = collapsed_token_stride(src, "src"), ds = collapsed_token_stride(dst, "dst");
  const float* c = nullptr;
  const float* s = nullptr;
  const void* p = nullptr;
  bool i64 = false;
  if (rot_dim > 0) {
    TORCH_CHECK(cos.has_value() && sin.has_value() && positions.has_value(), "rotation needs cos, sin and positions");
    check_f32(*cos, "cos");
    check_f32(*sin, "sin");
    TORCH_CHECK(positions->is_cuda() && positions->is_contiguous() && positions->numel() == tokens &&
                    (positions->scalar_type() == at::kLong || positions->scalar_type() == at::kInt),
                "positions must be contiguous CUDA int32/int64, one per token");
    TORCH_CHECK(cos->size(-1) * 2 == rot_dim, "cos/sin tables must be [max_pos, rot_dim/2]");
    c = cos->data_ptr<float>();
    s = sin->data_ptr<float>();
    p = positions->data_ptr();
    i64 = positions->scalar_type() == at::kLong;
  }
  c10::cuda::CUDAGuard guard(src.device());
  HB_CUDA_OK(hb::rope_apply(src.data_ptr(), dst.data_ptr(), c, s, p, i64, (int)tokens, (int)heads, (int)head_dim,
                            (int)rot_dim, ss, ds, interleaved, conjugate, cur_stream()));
}

at::Tensor gated_act_fwd(const at::Tensor& gate, const at::Tensor& up, int64_t kind) {
  TORCH_CHECK(gate.is_cuda() && gate.scalar_type() == at::kBFloat16 && gate.stride(-1) == 1);
  TORCH_CHECK(up.is_cuda() && up.scalar_type() == at::kBFloat16 && up.stride(-1) == 1);
  TORCH_CHECK(gate.sizes() == up.sizes(), "gate/up shapes differ");
  const int64_t row = gate.size(-1);
  at::Tensor g2 = gate.dim() == 2 ? gate : gate.reshape({-1, row});
  at::Tensor u2 = up.dim() == 2 ? up : up.reshape({-1, row});
  c10::cuda::CUDAGuard guard(gate.device());
  at::Tensor out = at::empty(gate.sizes(), gate.options());
  HB_CUDA_OK(hb::gated_act_fwd(g2.data_ptr(), u2.data_ptr(), out.data_ptr(), out.numel(), row,
                               g2.stride(0), u2.stride(0), (int)kind, cur_stream()));
  return out;
}

std::tuple<at::Tensor, at::Tensor> gated_act_bwd(const at::Tensor& gate, const at::Tensor& up,
                                                 const at::Tensor& dout, int64_t kind,
                                                 const c10::optional<at::Tensor>& dgate_out,
                                                 const c10::optional<at::Tensor>& dup_out) {
  const int64_t row = gate.size(-1);
  at::Tensor g2 = gate.dim() == 2 ? gate : gate.reshape({-1, row});
  at::Tensor u2 = up.dim() == 2 ? up : up.reshape({-1, row});
  check_bf16(dout, "dout");
  c10::cuda::CUDAGuard guard(gate.device());
  at::Tensor dg = dgate_out.has_value() ? *dgate_out : at::empty({g2.size(0), row}, gate.options());
  at::Tensor du = dup_out.has_value() ? *dup_out : at::empty({g2.size(0), row}, gate.options());
  TORCH_CHECK(dg.stride(-1) == 1 && du.stride(-1) == 1 && dg.dim() == 2 && du.dim() == 2);
  HB_CUDA_OK(hb::gated_act_bwd(g2.data_ptr(), u2.data_ptr(), dout.data_ptr(), dg.data_ptr(),
                               du.data_ptr(), dout.numel(), row, g2.stride(0), u2.stride(0),
                               dg.stride(0), du.stride(0), (int)kind, cur_stream()));
  return {dg, du};
}

// logits [rows, vocab] (bf16/fp32, row stride ld). Returns (loss, lse, zloss, entropy?) and
// writes the gradient into dlogits when given (may be the logits tensor itself).
std::vector<at::Tensor> cross_entropy(const at::Tensor& logits,
                                      const c10::optional<at::Tensor>& targets,
                                      const c10::optional<at::Tensor>& dlogits, int64_t ignore_index,
                                      double z_loss, double softcap, double logit_scale,
                                      double label_smoothing, double grad_scale,
                                      const c10::optional<at::Tensor>& grad_scale_t,
                                      const c10::optional<at::Tensor>& row_scale,
                                      bool want_entropy, int64_t vocab_start) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1);
  TORCH_CHECK(logits.scalar_type() == at::kBFloat16 || logits.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t rows = logits.size(0), vocab = logits.size(1);
  auto fopt = logits.options().dtype(at::kFloat);
  at::Tensor loss = at::empty({rows}, fopt), lse = at::empty({rows}, fopt),
             zl = at::empty({rows}, fopt);
  at::Tensor ent;
  if (want_entropy) ent = at::empty({rows}, fopt);
  hb::CEArgs a;
  a.logits = logits.data_ptr();
  a.logits_f32 = logits.scalar_type() == at::kFloat;
  if (targets.has_value()) {
    TORCH_CHECK(targets->is_cuda() && targets->scalar_type() == at::kLong &&
                targets->is_contiguous() && targets->numel() == rows);
    a.targets = targets->data_ptr<int64_t>();
  }
  a.loss = loss.data_ptr<float>();
  a.lse = lse.data_ptr<float>();
  a.zloss = zl.data_ptr<float>();
  a.entropy = want_entropy ? ent.data_ptr<float>() : nullptr;
  if (dlogits.has_value()) {
    TORCH_CHECK(dlogits->scalar_type() == logits.scalar_type() && dlogits->stride(1) == 1 &&
                dlogits->stride(0) == logits.stride(0) && dlogits->sizes() == logits.sizes());
    a.dlogits = dlogits->data_ptr();
  }
  if (grad_scale_t.has_value()) {
    check_f32(*grad_scale_t, "grad_scale_t");
    a.grad_scale_ptr = grad_scale_t->data_ptr<float>();
  }
  if (row_scale.has_value()) {
    check_f32(*row_scale, "row_scale");
    TORCH_CHECK(row_scale->numel() == rows);
    a.row_scale = row_scale->data_ptr<float>();
  }
  a.grad_scale = (float)grad_scale;
  a.rows = (int)rows;
  a.vocab = (int)vocab;
  a.ld = logits.stride(0);
  a.ignore_index = ignore_index;
  a.z_loss = (float)z_loss;
  a.softcap = (float)softcap;
  a.logit_scale = (float)logit_scale;
  a.label_smoothing = (float)label_smoothing;
  a.vocab_start = (int)vocab_start;
  HB_CUDA_OK(hb::cross_entropy_fwd(a, cur_stream()));
  std::vector<at::Tensor> out = {loss, lse, zl};
  if (want_entropy) out.push_back(ent);
  return out;
}

void logprob_entropy_bwd_(const at::Tensor& logits, const at::Tensor& targets, const at::Tensor& lse,
                          const c10::optional<at::Tensor>& entropy,
                          const c10::optional<at::Tensor>& g_logprob,
                          const c10::optional<at::Tensor>& g_entropy,
                          const c10::optional<at::Tensor>& row_scale, at::Tensor& dlogits,
                          int64_t ignore_index, double logit_scale, int64_t vocab_start) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1);
  TORCH_CHECK(logits.scalar_type() == at::kBFloat16 || logits.scalar_type() == at::kFloat);
  TORCH_CHECK(dlogits.scalar_type() == logits.scalar_type() && dlogits.stride(1) == 1 &&
              dlogits.stride(0) == logits.stride(0) && dlogits.sizes() == logits.sizes());
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous());
  check_f32(lse, "lse");
  c10::cuda::CUDAGuard guard(logits.device());
  hb::LogprobBwdArgs a;
  a.logits = logits.data_ptr();
  a.logits_f32 = logits.scalar_type() == at::kFloat;
  a.targets = targets.data_ptr<int64_t>();
  a.lse = lse.data_ptr<float>();
  if (entropy.has_value()) { check_f32(*entropy, "entropy"); a.entropy = entropy->data_ptr<float>(); }
  if (g_logprob.has_value()) { check_f32(*g_logprob, "g_logprob"); a.g_logprob = g_logprob->data_ptr<float>(); }
  if (g_entropy.has_value()) {
    check_f32(*g_entropy, "g_entropy");
    TORCH_CHECK(entropy.has_value(), "g_entropy needs the forward entropy");
    a.g_entropy = g_entropy->data_ptr<float>();
  }
  if (row_scale.has_value()) { check_f32(*row_scale, "row_scale"); a.row_scale = row_scale->data_ptr<float>(); }
  a.dlogits = dlogits.data_ptr();
  a.rows = (int)logits.size(0);
  a.vocab = (int)logits.size(1);
  a.ld = logits.stride(0);
  a.ignore_index = ignore_index;
  a.logit_scale = (float)logit_scale;
  a.vocab_start = (int)vocab_start;
  HB_CUDA_OK(hb::logprob_entropy_bwd(a, cur_stream()));
}

void adamw_(at::Tensor& master, at::Tensor& exp_avg, at::Tensor& exp_avg_sq, const at::Tensor& grad,
            const c10::optional<at::Tensor>& param_bf16, double lr, double beta1, double beta2,
            double eps, double weight_decay, int64_t step, double grad_scale,
            const c10::optional<at::Tensor>& grad_scale_t) {
  check_f32(master, "master");
  check_f32(exp_avg, "exp_avg");
  check_f32(exp_avg_sq, "exp_avg_sq");
  TORCH_CHECK(grad.is_cuda() && grad.is_contiguous() && grad.numel() == master.numel());
  TORCH_CHECK(grad.scalar_type() == at::kFloat || grad.scalar_type() == at::kBFloat16);
  c10::cuda::CUDAGuard guard(master.device());
  hb::AdamWArgs a;
  a.master = master.data_ptr<float>();
  a.exp_avg = exp_avg.data_ptr<float>();
  a.exp_avg_sq = exp_avg_sq.data_ptr<float>();
  a.grad = grad.data_ptr();
  a.grad_f32 = grad.scalar_type() == at::kFloat;
  if (param_bf16.has_value()) {
    check_bf16(*param_bf16, "param_bf16");
    TORCH_CHECK(param_bf16->numel() == master.numel());
    a.param_bf16 = param_bf16->data_ptr();
  }
  a.n = master.numel();
  a.lr = (float)lr; a.beta1 = (float)beta1; a.beta2 = (float)beta2; a.eps = (float)eps;
  a.weight_decay = (float)weight_decay;
  a.step = (int)step;
  a.grad_scale = (float)grad_scale;
  if (grad_scale_t.has_value()) {
    check_f32(*grad_scale_t, "grad_scale_t");
    a.grad_scale_ptr = grad_scale_t->data_ptr<float>();
  }
  HB_CUDA_OK(hb::adamw_step(a, cur_stream()));
}

void sumsq_(const at::Tensor& x, at::Tensor& out) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous());
  TORCH_CHECK(x.scalar_type() == at::kFloat || x.scalar_type() == at::kBFloat16);
  check_f32(out, "out");
  c10::cuda::CUDAGuard guard(x.device());
  HB_CUDA_OK(hb::sumsq(x.data_ptr(), x.scalar_type() == at::kFloat, x.numel(),
                       out.data_ptr<float>(), cur_stream()));
}

void clip_coef_(const at::Tensor& ss, double max_norm, at::Tensor& out) {
  check_f32(ss, "sumsq");
  check_f32(out, "out");
  TORCH_CHECK(out.numel() >= 2);
  c10::cuda::CUDAGuard guard(ss.device());
  HB_CUDA_OK(hb::clip_coef(ss.data_ptr<float>(), (float)max_norm, out.data_ptr<float>(), cur_stream()));
}

void cast_to_bf16_(const at::Tensor& src, at::Tensor& dst) {
  check_f32(src, "src");
  check_bf16(dst, "dst");
  TORCH_CHECK(src.numel() == dst.numel());
  c10::cuda::CUDAGuard guard(src.device());
  HB_CUDA_OK(hb::cast_f32_to_bf16(src.data_ptr<float>(), dst.data_ptr(), src.numel(), cur_stream()));
}

void cast_to_f32_(const at::Tensor& src, at::Tensor& dst, double scale, bool accumulate) {
  check_bf16(src, "src");
  check_f32(dst, "dst");
  TORCH_CHECK(src.numel() == dst.numel());
  c10::cuda::CUDAGuard guard(src.device());
  HB_CUDA_OK(hb::cast_bf16_to_f32(src.data_ptr(), dst.data_ptr<float>(), src.numel(), (float)scale,
                                  accumulate, cur_stream()));
}

std::tuple<at::Tensor, at::Tensor> gae(const at::Tensor& rewards, const at::Tensor& values,
                                       const c10::optional<at::Tensor>& mask, double gamma,
                                       double lam) {
  check_f32(rewards, "rewards");
  check_f32(values, "values");
  TORCH_CHECK(rewards.dim() == 2 && rewards.sizes() == values.sizes());
  if (mask.has_value()) {
    check_f32(*mask, "mask");
    TORCH_CHECK(mask->sizes() == rewards.sizes());
  }
  c10::cuda::CUDAGuard guard(rewards.device());
  at::Tensor adv = at::empty_like(rewards), ret = at::empty_like(rewards);
  HB_CUDA_OK(hb::gae(rewards.data_ptr<float>(), values.data_ptr<float>(),
                     mask.has_value() ? mask->data_ptr<float>() : nullptr, adv.data_ptr<float>(),
                     ret.data_ptr<float>(), (int)rewards.size(0), (int)rewards.size(1), (float)gamma,
                     (float)lam, cur_stream()));
  return {adv, ret};
}

// out[t] = a[t] * out[t -/+ 1] + b[t] * x[t] within each sequence of the packed row x[total, dim].
at::Tensor linear_scan(const at::Tensor& x, const at::Tensor& a, const at::Tensor& b, const at::Tensor& cu_seqlens,
                       bool reverse) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() &&
                  (x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kFloat),
              "x must be a contiguous CUDA bf16/fp32 [total, dim]");
  check_f32(a, "a");
  check_f32(b, "b");
  TORCH_CHECK(a.numel() == x.size(0) && b.numel() == x.size(0), "a and b hold one coefficient per row of x");
  TORCH_CHECK(cu_seqlens.is_cuda() && cu_seqlens.is_contiguous() && cu_seqlens.scalar_type() == at::kInt &&
                  cu_seqlens.numel() >= 1, "cu_seqlens must be contiguous CUDA int32");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor out = at::empty(x.sizes(), x.options().dtype(at::kFloat));
  HB_CUDA_OK(hb::linear_scan(x.data_ptr(), x.scalar_type() == at::kBFloat16, a.data_ptr<float>(),
                             b.data_ptr<float>(), cu_seqlens.data_ptr<int>(), (int)cu_seqlens.numel() - 1,
                             (int)x.size(1), reverse, out.data_ptr<float>(), cur_stream()));
  return out;
}

}  // namespace

void register_elementwise(pybind11::module_& m) {
  namespace py = pybind11;
  m.def("rmsnorm_fwd", &rmsnorm_fwd, py::arg("x"), py::arg("residual"), py::arg("w"),
        py::arg("eps"), py::arg("w_offset") = 0.0, py::arg("write_h") = true);
  m.def("rmsnorm_bwd", &rmsnorm_bwd, py::arg("dy"), py::arg("h"), py::arg("w"), py::arg("rstd"),
        py::arg("dres"), py::arg("w_offset") = 0.0);
  m.def("rope_", &rope_, py::arg("x"), py::arg("cos"), py::arg("sin"), py::arg("positions"),
        py::arg("rot_dim"), py::arg("interleaved"), py::arg("conjugate") = false);
  m.def("rope_copy", &rope_copy, py::arg("src"), py::arg("dst"), py::arg("cos"), py::arg("sin"),
        py::arg("positions"), py::arg("rot_dim"), py::arg("interleaved"), py::arg("conjugate") = false);
  m.def("gated_act_fwd", &gated_act_fwd, py::arg("gate"), py::arg("up"), py::arg("kind") = 0);
  m.def("gated_act_bwd", &gated_act_bwd, py::arg("gate"), py::arg("up"), py::arg("dout"),
        py::arg("kind") = 0, py::arg("dgate_out") = py::none(), py::arg("dup_out") = py::none());
  m.def("cross_entropy", &cross_entropy, py::arg("logits"), py::arg("targets"),
        py::arg("dlogits") = py::none(), py::arg("ignore_index") = -100, py::arg("z_loss") = 0.0,
        py::arg("softcap") = 0.0, py::arg("logit_scale") = 1.0, py::arg("label_smoothing") = 0.0,
        py::arg("grad_scale") = 1.0, py::arg("grad_scale_t") = py::none(),
        py::arg("row_scale") = py::none(), py::arg("want_entropy") = false,
        py::arg("vocab_start") = 0);
  m.def("logprob_entropy_bwd_", &logprob_entropy_bwd_, py::arg("logits"), py::arg("targets"),
        py::arg("lse"), py::arg("entropy"), py::arg("g_logprob"), py::arg("g_entropy"),
        py::arg("row_scale"), py::arg("dlogits"), py::arg("ignore_index") = -100,
        py::arg("logit_scale") = 1.0, py::arg("vocab_start") = 0);
  m.def("adamw_", &adamw_, py::arg("master"), py::arg("exp_avg"), py::arg("exp_avg_sq"),
        py::arg("grad"), py::arg("param_bf16"), py::arg("lr"), py::arg("beta1"), py::arg("beta2"),
        py::arg("eps"), py::arg("weight_decay"), py::arg("step"), py::arg("grad_scale") = 1.0,
        py::arg("grad_scale_t") = py::none());
  m.def("sumsq_", &sumsq_);
  m.def("clip_coef_", &clip_coef_);
  m.def("cast_to_bf16_", &cast_to_bf16_);
  m.def("cast_to_f32_", &cast_to_f32_, py::arg("src"), py::arg("dst"), py::arg("scale") = 1.0,
        py::arg("accumulate") = false);
  m.def("gae", &gae, py::arg("rewards"), py::arg("values"), py::arg("mask") = py::none(),
        py::arg("gamma") = 1.0, py::arg("lam") = 0.95);
  m.def("linear_scan", &linear_scan, py::arg("x"), py::arg("a"), py::arg("b"), py::arg("cu_seqlens"),
        py::arg("reverse") = false);
}
