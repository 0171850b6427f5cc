// One grouped-GEMM mode at a time on caller-owned tensors: the per-kernel entry points of the fused expert MLP.
//
// The layer executor (`FusedRank`) only ever runs the six modes as parts of a pass. This class launches ONE mode on
// tensors the caller provides, with the row groups of a single expert-major slice, so that every kernel can be
// tested against a plain reference on its own and used as a building block (`ops/fused_expert.py`). It mirrors the
// reference's kernel-level surface: gmm, gmm_swiglu, gmm_dswiglu, tgmm
// (src/chunked_moe/kernels/fused_expert.py:102-352).
//
// Rows: a slice holds at most `S` rows, expert after expert; `set_groups` takes the rows per expert as a device
// tensor and builds the tile tables on the device (no host synchronisation). Rows past the groups' total are padding:
// never read into a weight gradient, never written.
#pragma once

#include <torch/extension.h>

#include <cuda.h>
#include <cuda_runtime.h>

#include "../gemm/grouped_gemm.cuh"
#include "../plan/plan_kernel.cuh"

namespace cem {

class KernelRunner {
 public:
  KernelRunner(int L, int S, int stripe, int num_sms, bool cta_pairs);

  // rows per expert, int32 [L] on the device, sum <= S
  void set_groups(torch::Tensor group_rows);
  // act[S,F] = silu(x Wg) * (x Wu) from striped w_up [L,D,2F]; h [S,2F] (the rounded pre-activation) is optional
  void gmm_swiglu(torch::Tensor x, torch::Tensor w_up, torch::Tensor act, c10::optional<torch::Tensor> h);
  // out[S,N] = lhs[S,K] rhs[g]; rhs is [L,K,N], or [L,N,K] with transpose_rhs (no transpose is materialised)
  void gmm(torch::Tensor lhs, torch::Tensor rhs, torch::Tensor out, bool transpose_rhs);
  // dy[S,D] = w * g and dwp[S, D/256] = partial sums of <g, act W_down> per 256-column tile (y is never stored)
  void gmm_down_dw(torch::Tensor act, torch::Tensor w_down, torch::Tensor g, torch::Tensor row_w, torch::Tensor dy,
                   torch::Tensor dwp);
  // dh[S,2F] = SwiGLU'(h) * (dy W_down^T), w_down [L,F,D]
  void gmm_dswiglu(torch::Tensor dy, torch::Tensor w_down, torch::Tensor h, torch::Tensor dh);
  // out[g][M,N] = lhs[rows_g]^T rhs[rows_g] (bf16), lhs [S,M], rhs [S,N]
  void tgmm(torch::Tensor lhs, torch::Tensor rhs, torch::Tensor out);
  // Raises the first error a kernel recorded (synchronises the current stream).
  void check_status();

 private:
  GemmParams base() const;
  void launch(int mode, const GemmParams& p, const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap* c);
  int L_, S_, stripe_, num_sms_;
  bool pairs_;
  PlanLayout lay_;
  torch::Tensor plan_, counts_, status_, ones_, scratch_f32_, counter_, table_;
};

}  // namespace cem
