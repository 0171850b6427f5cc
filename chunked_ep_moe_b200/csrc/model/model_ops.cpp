// Tensor-level wrappers of the decoder's fused kernels (argument checks, allocation, stream).
#include "model_ops.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <stdexcept>
#include <string>

#include "model_kernels.cuh"
#include "router_kernels.cuh"

namespace cem {

namespace {

void need(bool cond, const char* msg) {
  if (!cond) throw std::runtime_error(std::string("model ops: ") + msg);
}

bool bf16_matrix(const torch::Tensor& t) {
  return t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.dim() == 2 && t.is_contiguous();
}

cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

}  // namespace

std::vector<torch::Tensor> add_rms_norm_fwd(torch::Tensor x, c10::optional<torch::Tensor> delta, torch::Tensor weight,
                                            double eps) {
  need(bf16_matrix(x), "x must be a contiguous CUDA bf16 matrix");
  const int64_t rows = x.size(0), cols = x.size(1);
  need(cols % 8 == 0 && cols <= 2048, "columns must be a multiple of 8, at most 2048");
  need(weight.is_cuda() && weight.scalar_type() == torch::kBFloat16 && weight.is_contiguous() && weight.numel() == cols,
       "weight must be a contiguous CUDA bf16 vector of `cols` elements");
  if (delta.has_value()) need(bf16_matrix(*delta) && delta->sizes() == x.sizes(), "delta must match x");
  const c10::cuda::CUDAGuard guard(x.device());
  torch::Tensor s = delta.has_value() ? torch::empty_like(x) : x;
  torch::Tensor y = torch::empty_like(x);
  torch::Tensor rstd = torch::empty({rows}, x.options().dtype(torch::kFloat32));
  launch_add_rms_norm_fwd(x.data_ptr(), delta.has_value() ? delta->data_ptr() : nullptr, weight.data_ptr(),
                          s.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), static_cast<int>(rows),
                          static_cast<int>(cols), static_cast<float>(eps), stream());
  return {s, y, rstd};
}

std::vector<torch::Tensor> add_rms_norm_bwd(torch::Tensor dy, c10::optional<torch::Tensor> ds_in, torch::Tensor s,
                                            torch::Tensor weight, torch::Tensor rstd) {
  need(bf16_matrix(dy) && bf16_matrix(s) && dy.sizes() == s.sizes(), "dy and s must be matching bf16 matrices");
  if (ds_in.has_value()) need(bf16_matrix(*ds_in) && ds_in->sizes() == s.sizes(), "ds_in must match s");
  const int64_t rows = s.size(0), cols = s.size(1);
  need(cols % 8 == 0 && cols <= 2048, "columns must be a multiple of 8, at most 2048");
  need(rstd.is_cuda() && rstd.scalar_type() == torch::kFloat32 && rstd.numel() == rows, "rstd must be fp32 [rows]");
  const c10::cuda::CUDAGuard guard(s.device());
  torch::Tensor ds = torch::empty_like(s);
  const int blocks = add_rms_norm_bwd_blocks(static_cast<int>(rows));
  torch::Tensor partial = torch::empty({blocks, cols}, s.options().dtype(torch::kFloat32));
  launch_add_rms_norm_bwd(dy.data_ptr(), ds_in.has_value() ? ds_in->data_ptr() : nullptr, s.data_ptr(),
                          weight.data_ptr(), rstd.data_ptr<float>(), ds.data_ptr(), partial.data_ptr<float>(),
                          static_cast<int>(rows), static_cast<int>(cols), stream());
  return {ds, partial.sum(0)};
}

std::vector<torch::Tensor> rope_qkv_fwd(torch::Tensor qkv, torch::Tensor cos_t, torch::Tensor sin_t) {
  need(qkv.is_cuda() && qkv.scalar_type() == torch::kBFloat16 && qkv.dim() == 5 && qkv.size(2) == 3 &&
           qkv.is_contiguous(),
       "qkv must be a contiguous CUDA bf16 [B, S, 3, H, hd] tensor");
  const int64_t B = qkv.size(0), S = qkv.size(1), H = qkv.size(3), hd = qkv.size(4);
  need(hd % 8 == 0, "head dimension must be a multiple of 8");
  need(cos_t.is_cuda() && cos_t.scalar_type() == torch::kFloat32 && cos_t.is_contiguous() && cos_t.dim() == 2 &&
           cos_t.size(0) >= S && cos_t.size(1) == hd / 2 && sin_t.sizes() == cos_t.sizes() && sin_t.is_contiguous() &&
           sin_t.scalar_type() == torch::kFloat32,
       "cos / sin must be contiguous CUDA fp32 [>= S, hd/2] tables");
  const c10::cuda::CUDAGuard guard(qkv.device());
  torch::Tensor q = torch::empty({B, H, S, hd}, qkv.options()), k = torch::empty_like(q), v = torch::empty_like(q);
  launch_rope_qkv(qkv.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), cos_t.data_ptr<float>(),
                  sin_t.data_ptr<float>(), static_cast<int>(B), static_cast<int>(S), static_cast<int>(H),
                  static_cast<int>(hd), false, stream());
  return {q, k, v};
}

torch::Tensor rope_qkv_bwd(torch::Tensor dq, torch::Tensor dk, torch::Tensor dv, torch::Tensor cos_t,
                           torch::Tensor sin_t) {
  need(dq.is_cuda() && dq.scalar_type() == torch::kBFloat16 && dq.dim() == 4 && dq.is_contiguous() &&
           dk.sizes() == dq.sizes() && dv.sizes() == dq.sizes() && dk.is_contiguous() && dv.is_contiguous() &&
           dk.scalar_type() == torch::kBFloat16 && dv.scalar_type() == torch::kBFloat16,
       "dq, dk, dv must be contiguous CUDA bf16 [B, H, S, hd] tensors");
  const int64_t B = dq.size(0), H = dq.size(1), S = dq.size(2), hd = dq.size(3);
  const c10::cuda::CUDAGuard guard(dq.device());
  torch::Tensor dqkv = torch::empty({B, S, 3, H, hd}, dq.options());
  launch_rope_qkv(dqkv.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), cos_t.data_ptr<float>(),
                  sin_t.data_ptr<float>(), static_cast<int>(B), static_cast<int>(S), static_cast<int>(H),
                  static_cast<int>(hd), true, stream());
  return dqkv;
}

std::vector<torch::Tensor> cross_entropy_fwd(torch::Tensor logits, torch::Tensor targets) {
  need(bf16_matrix(logits) && logits.size(1) % 8 == 0, "logits must be a contiguous CUDA bf16 [rows, cols % 8 == 0] matrix");
  need(targets.is_cuda() && targets.scalar_type() == torch::kInt64 && targets.is_contiguous() &&
           targets.numel() == logits.size(0),
       "targets must be a contiguous CUDA int64 vector of `rows` elements");
  const c10::cuda::CUDAGuard guard(logits.device());
  torch::Tensor loss = torch::empty({logits.size(0)}, logits.options().dtype(torch::kFloat32));
  torch::Tensor lse = torch::empty_like(loss);
  launch_cross_entropy_fwd(logits.data_ptr(), targets.data_ptr<int64_t>(), loss.data_ptr<float>(),
                           lse.data_ptr<float>(), static_cast<int>(logits.size(0)), static_cast<int>(logits.size(1)),
                           stream());
  return {loss, lse};
}

torch::Tensor cross_entropy_bwd(torch::Tensor logits, torch::Tensor targets, torch::Tensor lse,
                                torch::Tensor grad_scale) {
  need(bf16_matrix(logits), "logits must be a contiguous CUDA bf16 matrix");
  need(grad_scale.is_cuda() && grad_scale.scalar_type() == torch::kFloat32 && grad_scale.numel() == 1,
       "grad_scale must be a CUDA fp32 scalar");
  const c10::cuda::CUDAGuard guard(logits.device());
  torch::Tensor dlogits = torch::empty_like(logits);
  launch_cross_entropy_bwd(logits.data_ptr(), targets.data_ptr<int64_t>(), lse.data_ptr<float>(),
                           grad_scale.data_ptr<float>(), dlogits.data_ptr(), static_cast<int>(logits.size(0)),
                           static_cast<int>(logits.size(1)), stream());
  return dlogits;
}

torch::Tensor dense_swiglu_fwd(torch::Tensor gu) {
  need(bf16_matrix(gu) && gu.size(1) % 16 == 0, "gu must be a contiguous CUDA bf16 [rows, 2*ffn] matrix, ffn % 8 == 0");
  const c10::cuda::CUDAGuard guard(gu.device());
  torch::Tensor act = torch::empty({gu.size(0), gu.size(1) / 2}, gu.options());
  launch_dense_swiglu(gu.data_ptr(), nullptr, act.data_ptr(), static_cast<int>(gu.size(0)),
                      static_cast<int>(gu.size(1) / 2), false, stream());
  return act;
}

torch::Tensor dense_swiglu_bwd(torch::Tensor gu, torch::Tensor d_act) {
  need(bf16_matrix(gu) && gu.size(1) % 16 == 0, "gu must be a contiguous CUDA bf16 [rows, 2*ffn] matrix, ffn % 8 == 0");
  need(bf16_matrix(d_act) && d_act.size(0) == gu.size(0) && d_act.size(1) * 2 == gu.size(1),
       "d_act must be a contiguous CUDA bf16 [rows, ffn] matrix");
  const c10::cuda::CUDAGuard guard(gu.device());
  torch::Tensor d_gu = torch::empty_like(gu);
  launch_dense_swiglu(gu.data_ptr(), d_act.data_ptr(), d_gu.data_ptr(), static_cast<int>(gu.size(0)),
                      static_cast<int>(gu.size(1) / 2), true, stream());
  return d_gu;
}

std::vector<torch::Tensor> router_fwd(torch::Tensor logits, torch::Tensor bias, int64_t top_k, double scaling) {
  need(logits.is_cuda() && logits.scalar_type() == torch::kFloat32 && logits.dim() == 2 && logits.is_contiguous(),
       "logits must be a contiguous CUDA fp32 [tokens, experts] matrix");
  const int T = static_cast<int>(logits.size(0)), E = static_cast<int>(logits.size(1));
  need(router_supported(E, static_cast<int>(top_k)), "router kernel needs experts % 32 == 0, experts <= 256, top_k <= 32");
  need(bias.is_cuda() && bias.scalar_type() == torch::kFloat32 && bias.is_contiguous() && bias.numel() == E,
       "bias must be a contiguous CUDA fp32 vector of `experts` elements");
  const c10::cuda::CUDAGuard guard(logits.device());
  auto i32 = logits.options().dtype(torch::kInt32);
  torch::Tensor ids = torch::empty({T, top_k}, i32);
  torch::Tensor weights = torch::empty({T, top_k}, logits.options());
  torch::Tensor counts = torch::zeros({E}, i32);
  torch::Tensor partial = torch::empty({router_blocks(T), E}, logits.options());
  launch_router_fwd(logits.data_ptr<float>(), bias.data_ptr<float>(), ids.data_ptr<int>(), weights.data_ptr<float>(),
                    counts.data_ptr<int>(), partial.data_ptr<float>(), T, E, static_cast<int>(top_k),
                    static_cast<float>(scaling), stream());
  return {ids, weights, counts, partial};
}

torch::Tensor router_bwd(torch::Tensor logits, torch::Tensor ids, torch::Tensor d_weights, torch::Tensor d_prob,
                         double scaling) {
  need(logits.is_cuda() && logits.scalar_type() == torch::kFloat32 && logits.dim() == 2 && logits.is_contiguous(),
       "logits must be a contiguous CUDA fp32 [tokens, experts] matrix");
  const int T = static_cast<int>(logits.size(0)), E = static_cast<int>(logits.size(1));
  need(ids.is_cuda() && ids.scalar_type() == torch::kInt32 && ids.is_contiguous() && ids.dim() == 2 && ids.size(0) == T,
       "ids must be a contiguous CUDA int32 [tokens, top_k] matrix");
  const int top_k = static_cast<int>(ids.size(1));
  need(router_supported(E, top_k), "router kernel needs experts % 32 == 0, experts <= 256, top_k <= 32");
  need(d_weights.is_cuda() && d_weights.scalar_type() == torch::kFloat32 && d_weights.is_contiguous() &&
           d_weights.numel() == static_cast<int64_t>(T) * top_k,
       "d_weights must be a contiguous CUDA fp32 [tokens, top_k] matrix");
  need(d_prob.is_cuda() && d_prob.scalar_type() == torch::kFloat32 && d_prob.is_contiguous() && d_prob.numel() == E,
       "d_prob must be a contiguous CUDA fp32 vector of `experts` elements");
  const c10::cuda::CUDAGuard guard(logits.device());
  torch::Tensor d_logits = torch::empty_like(logits);
  launch_router_bwd(logits.data_ptr<float>(), ids.data_ptr<int>(), d_weights.data_ptr<float>(),
                    d_prob.data_ptr<float>(), d_logits.data_ptr<float>(), T, E, top_k, static_cast<float>(scaling),
                    stream());
  return d_logits;
}

}  // namespace cem
