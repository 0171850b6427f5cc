// Fused bandwidth-bound kernels of the decoder around the MoE layers (see model_kernels.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace cem {

// bf16 [rows, cols] tensors, cols a multiple of 8 and at most 2048; `delta` may be null (plain RMSNorm of x, `s_out`
// is then not written); `rstd` [rows] fp32.
void launch_add_rms_norm_fwd(const void* x, const void* delta, const void* w, void* s_out, void* y, float* rstd,
                             int rows, int cols, float eps, cudaStream_t stream);
// `ds_in` may be null. `dw_partial` is [add_rms_norm_bwd_blocks(rows), cols] fp32; its column sums are dW.
int add_rms_norm_bwd_blocks(int rows);
void launch_add_rms_norm_bwd(const void* dy, const void* ds_in, const void* s, const void* w, const float* rstd,
                             void* ds_out, float* dw_partial, int rows, int cols, cudaStream_t stream);
// Forward: qkv [B,S,3,H,hd] -> q, k rotated, v copied, each contiguous [B,H,S,hd]. Backward: the three gradients in
// [B,H,S,hd] -> d_qkv in the qkv layout (q and k rotated back). cos/sin: [S, hd/2] fp32; hd a multiple of 8.
void launch_rope_qkv(void* qkv, void* q, void* k, void* v, const float* cos_t, const float* sin_t, int B, int S, int H,
                     int hd, bool backward, cudaStream_t stream);
// bf16 logits [rows, cols] (cols a multiple of 8), int64 targets; per-row loss and log-sum-exp in fp32.
void launch_cross_entropy_fwd(const void* logits, const int64_t* targets, float* loss, float* lse, int rows, int cols,
                              cudaStream_t stream);
// dlogits = (softmax(logits) - onehot(target)) * *grad_scale, bf16 (may alias `logits`).
void launch_cross_entropy_bwd(const void* logits, const int64_t* targets, const float* lse, const float* grad_scale,
                              void* dlogits, int rows, int cols, cudaStream_t stream);

// bf16 gu [rows, 2*ffn] = [gate | up], ffn a multiple of 8. Forward: out = silu(gate) * up, [rows, ffn] (`d_act` unused).
// Backward: out = d_gu [rows, 2*ffn] from `d_act` [rows, ffn].
void launch_dense_swiglu(const void* gu, const void* d_act, void* out, int rows, int ffn, bool backward,
                         cudaStream_t stream);

}  // namespace cem
