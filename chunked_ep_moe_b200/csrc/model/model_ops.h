// Fused ops of the decoder around the MoE layers, on torch tensors (bound to Python in bindings.cpp).
#pragma once

#include <torch/extension.h>

#include <vector>

namespace cem {

// (s, y, rstd): s = x + delta (x itself without delta), y = RMSNorm(s) * weight.
std::vector<torch::Tensor> add_rms_norm_fwd(torch::Tensor x, c10::optional<torch::Tensor> delta, torch::Tensor weight,
                                            double eps);
// (ds, dweight): gradient w.r.t. s (= w.r.t. x and delta), including `ds_in` that flows into s from elsewhere.
std::vector<torch::Tensor> add_rms_norm_bwd(torch::Tensor dy, c10::optional<torch::Tensor> ds_in, torch::Tensor s,
                                            torch::Tensor weight, torch::Tensor rstd);
// (q, k, v) [B,H,S,hd] from qkv [B,S,3,H,hd]; q and k rotated.
std::vector<torch::Tensor> rope_qkv_fwd(torch::Tensor qkv, torch::Tensor cos_t, torch::Tensor sin_t);
torch::Tensor rope_qkv_bwd(torch::Tensor dq, torch::Tensor dk, torch::Tensor dv, torch::Tensor cos_t,
                           torch::Tensor sin_t);
// (loss per row, log-sum-exp per row), fp32.
std::vector<torch::Tensor> cross_entropy_fwd(torch::Tensor logits, torch::Tensor targets);
torch::Tensor cross_entropy_bwd(torch::Tensor logits, torch::Tensor targets, torch::Tensor lse,
                                torch::Tensor grad_scale);

// silu(gate) * up of gu = [gate | up] (bf16 [rows, 2*ffn]) and its backward (-> d_gu).
torch::Tensor dense_swiglu_fwd(torch::Tensor gu);
torch::Tensor dense_swiglu_bwd(torch::Tensor gu, torch::Tensor d_act);
// Sigmoid top-k router on fp32 logits [T, E]: (ids [T, K] int32, weights [T, K], counts [E] int32, per-block score
// sums [blocks, E]); backward: gradients of weights and of the score sums -> gradient of the logits.
std::vector<torch::Tensor> router_fwd(torch::Tensor logits, torch::Tensor bias, int64_t top_k, double scaling);
torch::Tensor router_bwd(torch::Tensor logits, torch::Tensor ids, torch::Tensor d_weights, torch::Tensor d_prob,
                         double scaling);

}  // namespace cem
