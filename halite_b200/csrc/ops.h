// Raw-pointer launchers of the memory-bound training / RL kernels (sm_100a).
// All activations are bf16 unless noted; statistics and reductions are fp32.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace hb {

// ---- RMSNorm (replaces the Triton kernels of nn/normalization.py:72,120 in the reference)
// h = x (+ residual); y = h * rsqrt(mean(h^2) + eps) * (w + w_offset); optionally writes h back.
cudaError_t rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* h_out,
                        float* rstd, int rows, int dim, float eps, float w_offset,
                        cudaStream_t stream);
// dx = rstd * (g - xhat * mean(g * xhat)) (+ dres), g = dy * (w + w_offset), xhat = h * rstd
// dw_partial[grid, dim] holds per-CTA partial sums of dy * xhat; returns grid size used.
cudaError_t rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd,
                        const void* dres, void* dx, float* dw_partial, int partial_rows, int rows,
                        int dim, float w_offset, cudaStream_t stream);
cudaError_t colsum_f32(const float* partial, int prows, int dim, void* out, bool out_bf16,
                       bool accumulate, cudaStream_t stream);

// ---- RoPE (replaces ops/rotary.py:14 of the reference). In place on x[tokens, heads, head_dim]
// (row stride `token_stride` elements), cos/sin tables [max_pos, rot_dim/2] fp32,
// positions int32/int64 per token. interleaved: pairs (2i, 2i+1); else (i, i + rot_dim/2).
cudaError_t rope_inplace(void* x, const float* cos, const float* sin, const void* positions,
                         bool pos_is_i64, int tokens, int heads, int head_dim, int rot_dim,
                         long token_stride, bool interleaved, bool conjugate, cudaStream_t stream);

// Out-of-place form: dst[token, head, :] = rotate(src[token, head, :]) with independent token strides
// (elements past rot_dim are copied; rot_dim = 0 is a strided copy). src == dst is the in-place case.
cudaError_t rope_apply(const void* src, void* dst, const float* cos, const float* sin, const void* positions,
                       bool pos_is_i64, int tokens, int heads, int head_dim, int rot_dim, long src_stride,
                       long dst_stride, bool interleaved, bool conjugate, cudaStream_t stream);

// ---- gated activations: out = act(gate) * up ; kind 0 = SiLU (SwiGLU), 1 = GELU tanh (GEGLU)
cudaError_t gated_act_fwd(const void* gate, const void* up, void* out, long n, long row, long gate_ld,
                          long up_ld, int kind, cudaStream_t stream);
cudaError_t gated_act_bwd(const void* gate, const void* up, const void* dout, void* dgate, void* dup,
                          long n, long row, long gate_ld, long up_ld, long dgate_ld, long dup_ld,
                          int kind, cudaStream_t stream);

// ---- cross entropy over rows of logits[rows, vocab] (bf16 or fp32). Writes per-row loss,
// lse, and (when dlogits != nullptr, may alias logits) the gradient
//   dlogits = grad_scale * (softmax * (1 + 2 z lse) - onehot)   for rows whose target != ignore
// softcap > 0 applies softcap * tanh(logit / softcap) first. logit_scale multiplies logits
// (1/temperature for the PPO log-prob path). entropy (optional) receives the row entropy.
struct CEArgs {
  const void* logits = nullptr;
  bool logits_f32 = false;
  const int64_t* targets = nullptr;
  float* loss = nullptr;      // [rows] (ce + z term), 0 for ignored rows
  float* lse = nullptr;       // [rows] optional
  float* zloss = nullptr;     // [rows] optional: z * lse^2 part alone
  float* entropy = nullptr;   // [rows] optional
  void* dlogits = nullptr;    // same dtype as logits, optional
  const float* grad_scale_ptr = nullptr;  // device scalar multiplier (optional)
  float grad_scale = 1.f;
  const float* row_scale = nullptr;  // [rows] optional per-row logit scale (1 / temperature)
  int rows = 0, vocab = 0;
  long ld = 0;
  int64_t ignore_index = -100;
  float z_loss = 0.f, softcap = 0.f, logit_scale = 1.f, label_smoothing = 0.f;
  int vocab_start = 0;  // first vocabulary id of this shard (vocab-parallel)
};
cudaError_t cross_entropy_fwd(const CEArgs& a, cudaStream_t stream);

// Gradient of per-row (log p[target], entropy) w.r.t. the logits; replaces the backward of the
// reference's Triton entropy kernel (nn/entropy.py:146) and of its log-prob cross entropy.
struct LogprobBwdArgs {
  const void* logits = nullptr;
  bool logits_f32 = false;
  const int64_t* targets = nullptr;
  const float* lse = nullptr;        // [rows] from the forward
  const float* entropy = nullptr;    // [rows] from the forward (needed when g_entropy is set)
  const float* g_logprob = nullptr;  // [rows] optional upstream gradient of log p[target]
  const float* g_entropy = nullptr;  // [rows] optional upstream gradient of the entropy
  const float* row_scale = nullptr;  // [rows] optional 1 / temperature
  void* dlogits = nullptr;           // may alias logits
  int rows = 0, vocab = 0;
  long ld = 0;
  int64_t ignore_index = -100;
  float logit_scale = 1.f;
  int vocab_start = 0;
};
cudaError_t logprob_entropy_bwd(const LogprobBwdArgs& a, cudaStream_t stream);

// ---- fused AdamW on a flat fp32 master shard with bf16 (or fp32) gradient, writes the bf16
// working copy in the same pass. grad_scale_ptr (device) multiplies the gradient
// (clip coefficient / loss scale); step is the 1-based step count.
struct AdamWArgs {
  float* master = nullptr;
  float* exp_avg = nullptr;
  float* exp_avg_sq = nullptr;
  const void* grad = nullptr;
  bool grad_f32 = true;
  void* param_bf16 = nullptr;  // optional working copy
  long n = 0;
  float lr = 0, beta1 = 0.9f, beta2 = 0.999f, eps = 1e-8f, weight_decay = 0;
  int step = 1;
  const float* grad_scale_ptr = nullptr;
  float grad_scale = 1.f;
};
cudaError_t adamw_step(const AdamWArgs& a, cudaStream_t stream);

// sum of squares of a flat buffer into *out (fp32, atomically accumulated; zero it first)
cudaError_t sumsq(const void* x, bool is_f32, long n, float* out, cudaStream_t stream);
// clip coefficient: out[0] = min(1, max_norm / (sqrt(sumsq[0]) + 1e-6)), out[1] = sqrt(sumsq)
cudaError_t clip_coef(const float* sumsq, float max_norm, float* out, cudaStream_t stream);

// dst(bf16) = src(fp32) * scale, or the reverse; flat
cudaError_t cast_f32_to_bf16(const float* src, void* dst, long n, cudaStream_t stream);
cudaError_t cast_bf16_to_f32(const void* src, float* dst, long n, float scale, bool accumulate,
                             cudaStream_t stream);

// ---- GAE reverse scan (replaces the Python loop of projects/ppo/trainer.py:200-213)
// rewards, values, mask: [B, T] fp32 (mask optional). adv, ret: [B, T] fp32.
cudaError_t gae(const float* rewards, const float* values, const float* mask, float* adv,
                float* ret, int B, int T, float gamma, float lam, cudaStream_t stream);

// ---- linear recurrence h[t] = a[t] * h[t-1] + b[t] * x[t] over each sequence of a packed row
// x[total, dim] (bf16 or fp32), a, b [total] fp32, cu_seqlens [n_seqs + 1] int32, out [total, dim] fp32;
// `reverse` runs every sequence from its last token to its first (the adjoint recurrence). Replaces the
// borrowed mamba-ssm scan of the reference's H-Net dechunk (transformers/models/hnet.py:112).
cudaError_t linear_scan(const void* x, bool x_bf16, const float* a, const float* b, const int* cu_seqlens,
                        int n_seqs, int dim, bool reverse, float* out, cudaStream_t stream);

}  // namespace hb
