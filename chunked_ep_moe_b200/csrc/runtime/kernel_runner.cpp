#include "kernel_runner.h"

#include <ATen/cuda/CUDAContext.h>

#include <stdexcept>
#include <string>

#include "fused_rank.h"
#include "tensor_map.h"

namespace cem {

namespace {

void need(bool cond, const std::string& msg) {
  if (!cond) throw std::runtime_error("KernelRunner: " + msg);
}

void need_bf16(const torch::Tensor& t, int64_t rows, int64_t cols, const char* name) {
  need(t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.dim() == 2 && t.is_contiguous() && t.size(0) == rows &&
           t.size(1) == cols,
       std::string(name) + " must be a contiguous CUDA bf16 [" + std::to_string(rows) + ", " + std::to_string(cols) +
           "] matrix");
}

void need_weights(const torch::Tensor& w, int64_t L, const char* name) {
  need(w.is_cuda() && w.scalar_type() == torch::kBFloat16 && w.dim() == 3 && w.is_contiguous() && w.size(0) == L,
       std::string(name) + " must be a contiguous CUDA bf16 [L, rows, cols] tensor");
}

cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

}  // namespace

KernelRunner::KernelRunner(int L, int S, int stripe, int num_sms, bool cta_pairs)
    : L_(L), S_(S), stripe_(stripe), num_sms_(num_sms), pairs_(cta_pairs && num_sms >= 2) {
  need(L >= 1 && L <= 1024, "1 <= L <= 1024");
  need(S >= 8 && S % 8 == 0, "S must be a positive multiple of 8");
  need(stripe == 32 || stripe == 64 || stripe == 128, "stripe must be 32, 64 or 128");
  lay_ = make_plan_layout(1, L, S, 1);
  auto i32 = torch::TensorOptions().device(torch::kCUDA).dtype(torch::kInt32);
  auto f32 = torch::TensorOptions().device(torch::kCUDA).dtype(torch::kFloat32);
  plan_ = torch::zeros({lay_.total}, i32);
  counts_ = torch::zeros({L}, i32);
  status_ = torch::zeros({8}, i32);
  ones_ = torch::ones({S}, f32);
  scratch_f32_ = torch::zeros({S}, f32);
  counter_ = torch::zeros({4}, i32);
  table_ = torch::zeros({4}, torch::TensorOptions().device(torch::kCUDA).dtype(torch::kInt64));
}

void KernelRunner::set_groups(torch::Tensor group_rows) {
  need(group_rows.is_cuda() && group_rows.scalar_type() == torch::kInt32 && group_rows.is_contiguous() &&
           group_rows.numel() == L_,
       "group_rows must be a contiguous CUDA int32 tensor of L elements");
  counts_.copy_(group_rows, /*non_blocking=*/true);
  PlanKernelParams pp{};
  pp.lay = lay_;
  pp.me = 0;
  pp.plan = plan_.data_ptr<int>();
  pp.counts = counts_.data_ptr<int>();
  pp.my_counts = counts_.data_ptr<int>();
  pp.spin_limit = 1;
  pp.status = reinterpret_cast<StatusBlock*>(status_.data_ptr());
  launch_plan_build(pp, stream());
}

GemmParams KernelRunner::base() const {
  GemmParams p{};
  p.plan = plan_.data_ptr<int>();
  p.lay = lay_;
  p.slice = 0;
  p.me = 0;
  p.stripe = stripe_;
  p.spin_limit = 1u << 20;
  p.mbar_limit = 20u * 1000u * 1000u;
  p.status = reinterpret_cast<StatusBlock*>(status_.data_ptr());
  return p;
}

void KernelRunner::launch(int mode, const GemmParams& p, const CUtensorMap& a, const CUtensorMap& b,
                          const CUtensorMap* c) {
  const CUtensorMap& out = c != nullptr ? *c : a;
  if (pairs_) launch_grouped_gemm_pair(mode, p, a, b, out, num_sms_, stream());
  else launch_grouped_gemm(mode, p, a, b, out, num_sms_, stream());
}

void KernelRunner::gmm_swiglu(torch::Tensor x, torch::Tensor w_up, torch::Tensor act, c10::optional<torch::Tensor> h) {
  need_weights(w_up, L_, "w_up");
  const int64_t D = w_up.size(1), F2 = w_up.size(2);
  need(D % 64 == 0 && F2 % 256 == 0 && (F2 / 2) % stripe_ == 0, "needs D % 64 == 0, 2F % 256 == 0, F % stripe == 0");
  need_bf16(x, S_, D, "x");
  need_bf16(act, S_, F2 / 2, "act");
  if (h.has_value()) need_bf16(*h, S_, F2, "h");
  GemmParams p = base();
  p.n_tiles = static_cast<int>(F2 / kBlockN);
  p.k_blocks = static_cast<int>(D / kBlockK);
  p.b_group_rows = static_cast<int>(D);
  p.out0 = reinterpret_cast<__nv_bfloat16*>(act.data_ptr());
  p.ld0 = static_cast<int>(F2 / 2);
  p.out1 = h.has_value() ? reinterpret_cast<__nv_bfloat16*>(h->data_ptr()) : nullptr;
  p.ld1 = static_cast<int>(F2);
  const CUtensorMap a = make_bf16_map_2d(x.data_ptr(), S_, D, 128);
  const CUtensorMap b = make_bf16_map_chunked(w_up.data_ptr(), static_cast<uint64_t>(L_) * D, F2, 64, pairs_ ? 2 : 4);
  launch(kModeSwiglu, p, a, b, nullptr);
}

void KernelRunner::gmm(torch::Tensor lhs, torch::Tensor rhs, torch::Tensor out, bool transpose_rhs) {
  need_weights(rhs, L_, "rhs");
  const int64_t K = transpose_rhs ? rhs.size(2) : rhs.size(1), N = transpose_rhs ? rhs.size(1) : rhs.size(2);
  need(K % 64 == 0 && N % 256 == 0, "needs K % 64 == 0 and N % 256 == 0");
  need_bf16(lhs, S_, K, "lhs");
  need_bf16(out, S_, N, "out");
  // One "rank": rows go back to where they came from, which is their own position in `out`.
  const int64_t ptrs[4] = {reinterpret_cast<int64_t>(out.data_ptr()), reinterpret_cast<int64_t>(counter_.data_ptr()),
                           reinterpret_cast<int64_t>(scratch_f32_.data_ptr()), 0};
  cudaMemcpyAsync(table_.data_ptr(), ptrs, sizeof(ptrs), cudaMemcpyHostToDevice, stream());
  GemmParams p = base();
  p.n_tiles = static_cast<int>(N / kBlockN);
  p.k_blocks = static_cast<int>(K / kBlockK);
  p.ld0 = static_cast<int>(N);
  p.peer_rows = reinterpret_cast<__nv_bfloat16* const*>(table_.data_ptr<int64_t>());
  p.peer_count = reinterpret_cast<uint32_t* const*>(table_.data_ptr<int64_t>() + 1);
  const CUtensorMap a = make_bf16_map_2d(lhs.data_ptr(), S_, K, 128);
  if (!transpose_rhs) {
    p.b_group_rows = static_cast<int>(K);
    p.row_w = ones_.data_ptr<float>();
    const CUtensorMap b = make_bf16_map_chunked(rhs.data_ptr(), static_cast<uint64_t>(L_) * K, N, 64, pairs_ ? 2 : 4);
    launch(kModeDownFwd, p, a, b, nullptr);
  } else {
    p.b_group_rows = static_cast<int>(N);
    p.peer_dw = reinterpret_cast<float* const*>(table_.data_ptr<int64_t>() + 2);
    p.dwp = nullptr;
    p.dwp_tiles = 0;  // no d_weight partials: the scalar that rides along is a plain zero
    const CUtensorMap b = make_bf16_map_2d(rhs.data_ptr(), static_cast<uint64_t>(L_) * N, K, pairs_ ? 128 : 256);
    launch(kModeDx, p, a, b, nullptr);
  }
}

void KernelRunner::gmm_down_dw(torch::Tensor act, torch::Tensor w_down, torch::Tensor g, torch::Tensor row_w,
                               torch::Tensor dy, torch::Tensor dwp) {
  need_weights(w_down, L_, "w_down");
  const int64_t F = w_down.size(1), D = w_down.size(2);
  need(F % 64 == 0 && D % 256 == 0, "needs F % 64 == 0 and D % 256 == 0");
  need_bf16(act, S_, F, "act");
  need_bf16(g, S_, D, "g");
  need_bf16(dy, S_, D, "dy");
  need(row_w.is_cuda() && row_w.scalar_type() == torch::kFloat32 && row_w.is_contiguous() && row_w.numel() == S_,
       "row_w must be a contiguous CUDA fp32 tensor of S elements");
  need(dwp.is_cuda() && dwp.scalar_type() == torch::kFloat32 && dwp.is_contiguous() && dwp.dim() == 2 &&
           dwp.size(0) == S_ && dwp.size(1) == D / kBlockN,
       "dwp must be a contiguous CUDA fp32 [S, D/256] tensor");
  GemmParams p = base();
  p.n_tiles = static_cast<int>(D / kBlockN);
  p.k_blocks = static_cast<int>(F / kBlockK);
  p.b_group_rows = static_cast<int>(F);
  p.row_w = row_w.data_ptr<float>();
  p.in0 = reinterpret_cast<const __nv_bfloat16*>(g.data_ptr());
  p.out0 = reinterpret_cast<__nv_bfloat16*>(dy.data_ptr());
  p.ld0 = static_cast<int>(D);
  p.dwp = dwp.data_ptr<float>();
  p.dwp_tiles = static_cast<int>(D / kBlockN);
  const CUtensorMap a = make_bf16_map_2d(act.data_ptr(), S_, F, 128);
  const CUtensorMap b = make_bf16_map_chunked(w_down.data_ptr(), static_cast<uint64_t>(L_) * F, D, 64, pairs_ ? 2 : 4);
  launch(kModeDownDw, p, a, b, nullptr);
}

void KernelRunner::gmm_dswiglu(torch::Tensor dy, torch::Tensor w_down, torch::Tensor h, torch::Tensor dh) {
  need_weights(w_down, L_, "w_down");
  const int64_t F = w_down.size(1), D = w_down.size(2);
  need(D % 64 == 0 && F % 256 == 0 && F % stripe_ == 0, "needs D % 64 == 0, F % 256 == 0, F % stripe == 0");
  need_bf16(dy, S_, D, "dy");
  need_bf16(h, S_, 2 * F, "h");
  need_bf16(dh, S_, 2 * F, "dh");
  GemmParams p = base();
  p.n_tiles = static_cast<int>(F / kBlockN);
  p.k_blocks = static_cast<int>(D / kBlockK);
  p.b_group_rows = static_cast<int>(F);
  p.in0 = reinterpret_cast<const __nv_bfloat16*>(h.data_ptr());
  p.out0 = reinterpret_cast<__nv_bfloat16*>(dh.data_ptr());
  p.ld0 = static_cast<int>(2 * F);
  const CUtensorMap a = make_bf16_map_2d(dy.data_ptr(), S_, D, 128);
  const CUtensorMap b = make_bf16_map_2d(w_down.data_ptr(), static_cast<uint64_t>(L_) * F, D, pairs_ ? 128 : 256);
  launch(kModeDswiglu, p, a, b, nullptr);
}

void KernelRunner::tgmm(torch::Tensor lhs, torch::Tensor rhs, torch::Tensor out) {
  need(lhs.dim() == 2 && rhs.dim() == 2, "lhs and rhs must be matrices");
  const int64_t M = lhs.size(1), N = rhs.size(1);
  need(M % 256 == 0 && N % 256 == 0, "needs M % 256 == 0 and N % 256 == 0");
  need_bf16(lhs, S_, M, "lhs");
  need_bf16(rhs, S_, N, "rhs");
  need(out.is_cuda() && out.scalar_type() == torch::kBFloat16 && out.is_contiguous() && out.dim() == 3 &&
           out.size(0) == L_ && out.size(1) == M && out.size(2) == N,
       "out must be a contiguous CUDA bf16 [L, M, N] tensor");
  GemmParams p = base();
  p.m_tiles = static_cast<int>(M / kBlockM);
  p.n_tiles = static_cast<int>(N / kBlockN);
  p.carry_in = nullptr;   // one slice: every group begins and ends in it, the carry is never touched
  p.carry_out = nullptr;
  p.grad_out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  const CUtensorMap a = make_bf16_map_chunked(lhs.data_ptr(), S_, M, 64, 2);
  const CUtensorMap b = make_bf16_map_chunked(rhs.data_ptr(), S_, N, 64, pairs_ ? 2 : 4);
  const CUtensorMap c = make_bf16_map_2d(out.data_ptr(), static_cast<uint64_t>(L_) * M, N, 32);
  launch(kModeTgmm, p, a, b, &c);
}

void KernelRunner::check_status() {
  int32_t host[8];
  cudaStream_t st = stream();
  cudaMemcpyAsync(host, status_.data_ptr(), sizeof(host), cudaMemcpyDeviceToHost, st);
  cudaStreamSynchronize(st);
  if (host[0] != 0) {
    const std::string message = format_status(std::vector<int64_t>(host, host + 8), 0);
    cudaMemsetAsync(status_.data_ptr(), 0, sizeof(host), st);
    cudaStreamSynchronize(st);
    throw std::runtime_error(message);
  }
}

}  // namespace cem
