#include "fused_rank.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>

#include "tensor_map.h"

namespace cem {

namespace {

constexpr int kExpandSms = 12;  // SMs the up-projection GEMM leaves to the fp8 expansion kernel

inline void cuda_check(cudaError_t err, const char* what) {
  if (err != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(err));
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

inline cudaStream_t current_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void expect(bool cond, const std::string& msg) {
  if (!cond) throw std::runtime_error(msg);
}

void expect_bf16_2d(const torch::Tensor& t, int64_t cols, const char* name) {
  expect(t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.dim() == 2 && t.size(1) == cols && t.is_contiguous(),
         std::string(name) + " must be a contiguous CUDA bf16 matrix with " + std::to_string(cols) + " columns");
}

void expect_i32(const torch::Tensor& t, int64_t min_numel, const char* name) {
  expect(t.is_cuda() && t.scalar_type() == torch::kInt32 && t.is_contiguous() && t.numel() >= min_numel,
         std::string(name) + " must be a contiguous CUDA int32 tensor with at least " + std::to_string(min_numel) +
             " elements");
}

const char* status_name(int code) {
  switch (code) {
    case kStatusMbarTimeout: return "pipeline barrier timed out";
    case kStatusArrivalTimeout: return "dispatched rows never arrived";
    case kStatusCreditTimeout: return "a receiver never released its slice buffer";
    case kStatusReturnTimeout: return "combined rows never came back";
    case kStatusBadIndex: return "index check failed";
    case kStatusTrafficTimeout: return "a peer's traffic-matrix row never arrived";
    default: return "unknown";
  }
}

}  // namespace

ArenaLayout make_arena_layout(int P, int L, int S, int D, int tk_cap, bool fp8) {
  ArenaLayout a{};
  size_t o = 0;
  auto take = [&](size_t bytes) { size_t at = o; o = align_up(o + bytes, 1024); return at; };
  a.xbuf = take(2ull * S * D * 2);
  a.gbuf = take(2ull * S * D * 2);
  a.wbuf = take(2ull * S * 4);
  a.xq = take(fp8 ? 2ull * S * D : 0);
  a.gq = take(fp8 ? 2ull * S * D : 0);
  a.xs = take(fp8 ? 2ull * S * (D / 128) * 4 : 0);
  a.gs = take(fp8 ? 2ull * S * (D / 128) * 4 : 0);
  a.ret = take(static_cast<size_t>(tk_cap) * D * 2);
  a.dw_rows = take(static_cast<size_t>(tk_cap) * 4);
  a.arrive = take(static_cast<size_t>(P) * L * 4);
  a.credit = take(static_cast<size_t>(P) * 4);
  a.ret_count = take(4);
  a.traffic = take(2ull * P * P * L * 4);
  a.traffic_flags = take(2ull * P * 4);
  a.total = o;
  return a;
}

FusedRank::FusedRank(int P, int L, int me, int S, int D, int F, int K, int stripe, int tk_cap, int max_slices,
                     int num_sms, bool fp8, int64_t arena, std::vector<int64_t> peer_arenas, bool use_comm_stream,
                     int64_t spin_limit, int put_blocks, bool cta_pairs, bool tgmm_pairs)
    : P_(P), L_(L), me_(me), S_(S), D_(D), F_(F), K_(K), stripe_(stripe), tk_cap_(tk_cap), max_slices_(max_slices),
      num_sms_(num_sms), put_blocks_(put_blocks), fp8_(fp8), use_comm_stream_(use_comm_stream),
      cta_pairs_(cta_pairs && num_sms >= 2), tgmm_pairs_(tgmm_pairs && num_sms >= 2) {
  expect(P >= 1 && L >= 1 && me >= 0 && me < P, "bad rank geometry");
  expect(static_cast<int>(peer_arenas.size()) == P, "need one arena pointer per rank");
  expect(P <= 32, "at most 32 expert-parallel ranks (one warp lane watches one source)");
  expect(P * L <= 1024, "at most 1024 experts");
  expect(D % 256 == 0, "fused kernels need D % 256 == 0");
  expect(F % 256 == 0, "fused kernels need F % 256 == 0");
  expect(stripe == 32 || stripe == 64 || stripe == 128, "fused kernels need stripe_width in {32, 64, 128}");
  expect(S % 8 == 0 && S >= 8, "fused kernels need slice_size % 8 == 0");
  expect(!fp8 || D % 128 == 0, "fp8 wire needs D % 128 == 0");
  spin_limit_ = static_cast<uint32_t>(spin_limit);
  if (const char* v = std::getenv("CEM_GEMM_EXCLUSIVE_SM")) g_gemm_extra_smem = std::atoi(v) != 0 ? 1024 : 0;
  if (const char* v = std::getenv("CEM_PAIR_SUSPEND")) g_pair_suspend_waits = std::atoi(v) != 0 ? 1 : 0;
  if (const char* v = std::getenv("CEM_RET_BLOCKED")) ret_blocked_ = std::atoi(v) != 0;
  if (const char* v = std::getenv("CEM_RET_LSU")) ret_lsu_ = std::atoi(v) != 0;
  mbar_limit_ = 20u * 1000u * 1000u;  // microseconds: longer than any legitimate wait on another rank
  lay_ = make_plan_layout(P, L, S, max_slices);
  arena_lay_ = make_arena_layout(P, L, S, D, tk_cap, fp8);
  arena_ = reinterpret_cast<uint8_t*>(arena);
  for (int64_t p : peer_arenas) peers_.push_back(reinterpret_cast<uint8_t*>(p));

  auto bf16 = torch::TensorOptions().device(torch::kCUDA).dtype(torch::kBFloat16);
  auto f32 = torch::TensorOptions().device(torch::kCUDA).dtype(torch::kFloat32);
  auto i32 = torch::TensorOptions().device(torch::kCUDA).dtype(torch::kInt32);
  for (int q = 0; q < 2; ++q) {  // double buffered by slice parity: two slices are in flight at a time
    act_[q] = torch::zeros({S, F}, bf16);
    h_[q] = torch::zeros({S, 2 * F}, bf16);
    dy_[q] = torch::zeros({S, D}, bf16);
    dh_[q] = torch::zeros({S, 2 * F}, bf16);
    dwp_[q] = torch::zeros({S, D / 256}, f32);
  }
  carry_up_ = torch::zeros({2, D, 2 * F}, f32);
  carry_down_ = torch::zeros({2, F, D}, f32);
  pass_base_ = torch::zeros({P * L}, i32);
  ready_ = torch::zeros({L}, i32);
  ready_base_ = torch::zeros({L}, i32);
  ready_total_ = torch::zeros({L}, i32);
  expected_total_ = torch::zeros({P * L}, i32);
  status_ = torch::zeros({8}, i32);
  my_counts_ = torch::zeros({P * L}, i32);
  sort_scratch_ = torch::zeros({static_cast<int64_t>(expert_sort_scratch_ints(tk_cap, P * L))}, i32);

  // Pointer tables: row t holds, for every rank r, the address of buffer t inside r's arena.
  std::vector<int64_t> host(static_cast<size_t>(kNumTables) * P);
  const size_t traffic_half = static_cast<size_t>(P) * P * L * 4, flags_half = static_cast<size_t>(P) * 4;
  for (int r = 0; r < P; ++r) {
    auto at = [&](size_t off) { return reinterpret_cast<int64_t>(peers_[r] + off); };
    host[kTabX * P + r] = at(arena_lay_.xbuf);
    host[kTabG * P + r] = at(arena_lay_.gbuf);
    host[kTabW * P + r] = at(arena_lay_.wbuf);
    host[kTabXq * P + r] = at(arena_lay_.xq);
    host[kTabGq * P + r] = at(arena_lay_.gq);
    host[kTabXs * P + r] = at(arena_lay_.xs);
    host[kTabGs * P + r] = at(arena_lay_.gs);
    host[kTabArrive * P + r] = at(arena_lay_.arrive);
    host[kTabRet * P + r] = at(arena_lay_.ret);
    host[kTabDw * P + r] = at(arena_lay_.dw_rows);
    host[kTabCount * P + r] = at(arena_lay_.ret_count);
    host[kTabCredit * P + r] = at(arena_lay_.credit);
    host[kTabTraffic0 * P + r] = at(arena_lay_.traffic);
    host[kTabTraffic1 * P + r] = at(arena_lay_.traffic + traffic_half);
    host[kTabTflags0 * P + r] = at(arena_lay_.traffic_flags);
    host[kTabTflags1 * P + r] = at(arena_lay_.traffic_flags + flags_half);
  }
  tables_ = torch::from_blob(host.data(), {static_cast<int64_t>(kNumTables), P}, torch::kInt64).clone().to(torch::kCUDA);

  // TMA descriptors of the local buffers. K-major A tiles are 128 rows, MN-major tiles 64 rows (k) of several
  // 64-column chunks brought by one 3-D copy (a CTA of a pair loads half of the 256-wide column tile).
  const uint32_t mn_chunks_b = tgmm_pairs_ ? 2 : 4;  // the MN-major maps of local buffers feed the weight-gradient mode
  for (int b = 0; b < 2; ++b) {
    const void* xb = arena_ + arena_lay_.xbuf + static_cast<size_t>(b) * S * D * 2;
    map_x_k_[b] = make_bf16_map_2d(xb, S, D, 128);
    map_x_mn_[b] = make_bf16_map_chunked(xb, S, D, 64, 2);  // weight-gradient lhs: 128 columns per tile
  }
  for (int q = 0; q < 2; ++q) {
    map_act_k_[q] = make_bf16_map_2d(act_[q].data_ptr(), S, F, 128);
    map_act_mn_[q] = make_bf16_map_chunked(act_[q].data_ptr(), S, F, 64, 2);
    map_dy_k_[q] = make_bf16_map_2d(dy_[q].data_ptr(), S, D, 128);
    map_dy_mn_[q] = make_bf16_map_chunked(dy_[q].data_ptr(), S, D, 64, mn_chunks_b);  // weight-gradient rhs
    map_dh_k_[q] = make_bf16_map_2d(dh_[q].data_ptr(), S, 2 * F, 128);
    map_dh_mn_[q] = make_bf16_map_chunked(dh_[q].data_ptr(), S, 2 * F, 64, mn_chunks_b);
  }

  if (use_comm_stream_) {
    // The put and expansion kernels feed kernels that wait for them: their blocks go first when SMs free up.
    int prio_low = 0, prio_high = 0;
    cuda_check(cudaDeviceGetStreamPriorityRange(&prio_low, &prio_high), "stream priority range");
    if (const char* v = std::getenv("CEM_COMM_PRIORITY")) {
      if (std::atoi(v) == 0) prio_high = prio_low;  // measurement knob: comm streams at the default priority
    }
    cuda_check(cudaStreamCreateWithPriority(&comm_stream_, cudaStreamNonBlocking, prio_high), "comm stream");
    cuda_check(cudaStreamCreateWithFlags(&aux_stream_, cudaStreamNonBlocking), "aux stream");
    for (int q = 0; q < 2; ++q) cuda_check(cudaStreamCreateWithFlags(&chain_[q], cudaStreamNonBlocking), "chain stream");
    if (fp8_) cuda_check(cudaStreamCreateWithPriority(&expand_stream_, cudaStreamNonBlocking, prio_high), "expand stream");
  }
  for (int i = 0; i < 4; ++i) cuda_check(cudaEventCreateWithFlags(&ev_expand_[i], cudaEventDisableTiming), "event");
  for (int q = 0; q < 2; ++q)
    for (cudaEvent_t* e : {&ev_down_[q], &ev_dd_[q], &ev_ds_[q], &ev_dx_[q], &ev_tgd_[q], &ev_tgu_[q]})
      cuda_check(cudaEventCreateWithFlags(e, cudaEventDisableTiming), "event");
  cuda_check(cudaEventCreateWithFlags(&ev_pass_, cudaEventDisableTiming), "event");
  cuda_check(cudaEventCreateWithFlags(&ev_header_, cudaEventDisableTiming | cudaEventBlockingSync), "event");
  for (int i = 0; i < 4; ++i) {
    cuda_check(cudaEventCreateWithFlags(&ev_put_[i], cudaEventDisableTiming), "event");
    cuda_check(cudaEventCreateWithFlags(&ev_done_[i], cudaEventDisableTiming), "event");
  }
  cuda_check(cudaMallocHost(reinterpret_cast<void**>(&host_header_), 24 * sizeof(int32_t)), "pinned header");
  std::memset(host_header_, 0, 24 * sizeof(int32_t));
}

FusedRank::~FusedRank() {
  if (comm_stream_) cudaStreamDestroy(comm_stream_);
  if (aux_stream_) cudaStreamDestroy(aux_stream_);
  if (expand_stream_) cudaStreamDestroy(expand_stream_);
  for (int i = 0; i < 4; ++i)
    if (ev_expand_[i]) cudaEventDestroy(ev_expand_[i]);
  for (int q = 0; q < 2; ++q) {
    if (chain_[q]) cudaStreamDestroy(chain_[q]);
    for (cudaEvent_t e : {ev_down_[q], ev_dd_[q], ev_ds_[q], ev_dx_[q], ev_tgd_[q], ev_tgu_[q]})
      if (e) cudaEventDestroy(e);
  }
  if (ev_pass_) cudaEventDestroy(ev_pass_);
  if (ev_header_) cudaEventDestroy(ev_header_);
  for (int i = 0; i < 4; ++i) {
    if (ev_put_[i]) cudaEventDestroy(ev_put_[i]);
    if (ev_done_[i]) cudaEventDestroy(ev_done_[i]);
  }
  if (host_header_) cudaFreeHost(host_header_);
}

void FusedRank::check_status() {
  cudaStream_t st = current_stream();
  cuda_check(cudaMemcpyAsync(host_header_ + 16, status_.data_ptr(), 8 * sizeof(int32_t), cudaMemcpyDeviceToHost, st),
             "status copy");
  cuda_check(cudaStreamSynchronize(st), "status sync");
  const int32_t* s = host_header_ + 16;
  if (s[0] != 0) {
    const std::string message = format_status(std::vector<int64_t>(s, s + 8), me_);
    cuda_check(cudaMemsetAsync(status_.data_ptr(), 0, 8 * sizeof(int32_t), st), "status clear");
    cuda_check(cudaStreamSynchronize(st), "status clear sync");
    throw std::runtime_error(message);
  }
}

std::string format_status(const std::vector<int64_t>& s, int rank) {
  if (s.size() < 8) return "chunked_moe fused path: malformed status block";
  char buf[512];
  std::snprintf(buf, sizeof(buf),
                "chunked_moe fused path: %s (code %lld, kernel %lld, mode %lld, slice/tile %lld, detail %lld, "
                "expected %llu, seen %llu, block %lld, rank %d)",
                status_name(static_cast<int>(s[0])), static_cast<long long>(s[0]), static_cast<long long>(s[1]),
                static_cast<long long>(s[2]), static_cast<long long>(s[3]), static_cast<long long>(s[4]),
                static_cast<unsigned long long>(static_cast<uint32_t>(s[5])),
                static_cast<unsigned long long>(static_cast<uint32_t>(s[6])), static_cast<long long>(s[7]), rank);
  return std::string(buf);
}

void FusedRank::sort_only(torch::Tensor expert_ids, torch::Tensor order, torch::Tensor inv_order,
                          torch::Tensor my_counts) {
  const int64_t tk = expert_ids.numel();
  expect(tk <= tk_cap_, "T*K exceeds the workspace capacity");
  expect_i32(expert_ids, tk, "expert_ids");
  expect_i32(order, tk, "order");
  expect_i32(inv_order, tk, "inv_order");
  expect_i32(my_counts, P_ * L_, "my_counts");
  launch_expert_sort(expert_ids.data_ptr<int>(), static_cast<int>(tk), P_ * L_, order.data_ptr<int>(),
                     inv_order.data_ptr<int>(), my_counts.data_ptr<int>(), sort_scratch_.data_ptr<int>(),
                     current_stream(), reinterpret_cast<StatusBlock*>(status_.data_ptr()));
  launches_ += 3;
}

int64_t FusedRank::begin_forward_async(torch::Tensor expert_ids, torch::Tensor plan, torch::Tensor order,
                                       torch::Tensor inv_order, torch::Tensor counts, bool counts_prefilled) {
  cudaStream_t st = current_stream();
  const int64_t tk = expert_ids.numel();
  expect(tk <= tk_cap_, "T*K exceeds the workspace capacity");
  expect_i32(plan, lay_.total, "plan");
  PlanKernelParams pp{};
  pp.lay = lay_;
  pp.me = me_;
  pp.plan = plan.data_ptr<int>();
  pp.spin_limit = spin_limit_;
  pp.status = reinterpret_cast<StatusBlock*>(status_.data_ptr());
  if (counts_prefilled) {
    expect_i32(counts, static_cast<int64_t>(P_) * P_ * L_, "counts");
    pp.counts = counts.data_ptr<int>();
    pp.my_counts = counts.data_ptr<int>() + static_cast<size_t>(me_) * P_ * L_;
    pp.peer_counts = nullptr;
    pp.peer_flags = nullptr;
    pp.flags = nullptr;
    pp.epoch = 0;
  } else {
    sort_only(expert_ids, order, inv_order, my_counts_);
    const uint32_t epoch = ++fwd_epoch_;
    const int parity = static_cast<int>(epoch & 1u);
    pp.my_counts = my_counts_.data_ptr<int>();
    pp.counts = reinterpret_cast<int*>(arena_ + arena_lay_.traffic + static_cast<size_t>(parity) * P_ * P_ * L_ * 4);
    pp.peer_counts = table<int>(parity ? kTabTraffic1 : kTabTraffic0);
    pp.peer_flags = table<uint32_t>(parity ? kTabTflags1 : kTabTflags0);
    pp.flags = reinterpret_cast<const uint32_t*>(arena_ + arena_lay_.traffic_flags + static_cast<size_t>(parity) * P_ * 4);
    pp.epoch = epoch;
  }
  launch_plan_build(pp, st);
  ++launches_;
  // Header and status follow the plan kernel to the host; nobody waits here.
  cuda_check(cudaMemcpyAsync(host_header_, plan.data_ptr(), 16 * sizeof(int32_t), cudaMemcpyDeviceToHost, st),
             "plan header copy");
  cuda_check(cudaMemcpyAsync(host_header_ + 16, status_.data_ptr(), 8 * sizeof(int32_t), cudaMemcpyDeviceToHost, st),
             "status copy");
  cuda_check(cudaEventRecord(ev_header_, st), "event record");
  begin_backward(plan, max_slices_, tk);  // any slice below the workspace's capacity may be launched until resolved
  return last_slices_ < 0 ? -1 : std::min<int64_t>(last_slices_, max_slices_);
}

int64_t FusedRank::resolve_slices() {
  cuda_check(cudaEventSynchronize(ev_header_), "plan header wait");
  const int32_t* st = host_header_ + 16;
  if (st[0] != 0) {
    const std::string message = format_status(std::vector<int64_t>(st, st + 8), me_);
    cudaStream_t cur = current_stream();
    cuda_check(cudaStreamSynchronize(cur), "status sync");  // what was launched on the guess ends (at once) first
    cuda_check(cudaMemsetAsync(status_.data_ptr(), 0, 8 * sizeof(int32_t), cur), "status clear");
    cuda_check(cudaStreamSynchronize(cur), "status clear sync");
    throw std::runtime_error(message);
  }
  expect(host_header_[4] == 0, "routing needs more slices than the workspace was sized for (max_slices)");
  expect(host_header_[5] == cur_rows_, "the routing plan does not account for every token copy");
  last_slices_ = host_header_[0];
  return last_slices_;
}

void FusedRank::set_pass_slices(int64_t launched) {
  expect(launched >= 0 && launched <= max_slices_, "slice count exceeds the workspace");
  cur_slices_ = launched;
}

void FusedRank::set_mbar_limit_us(int64_t us) {
  expect(us > 0 && us <= 600ll * 1000 * 1000, "barrier limit must be between 1 us and 600 s");
  mbar_limit_ = static_cast<uint32_t>(us);
}

int64_t FusedRank::begin_forward(torch::Tensor expert_ids, torch::Tensor plan, torch::Tensor order,
                                 torch::Tensor inv_order, torch::Tensor counts, bool counts_prefilled) {
  begin_forward_async(expert_ids, plan, order, inv_order, counts, counts_prefilled);
  const int64_t n = resolve_slices();
  set_pass_slices(n);
  return n;
}


int64_t FusedRank::begin_backward(torch::Tensor plan, int64_t known_slices, int64_t known_rows) {
  cudaStream_t st = current_stream();
  expect_i32(plan, lay_.total, "plan");
  if (known_slices >= 0 && known_rows >= 0) {
    // The caller kept what the forward of this plan read back: no device-to-host copy, no synchronisation, so the
    // host keeps running ahead of the device through the whole backward. (A recorded kernel error then surfaces at
    // the next synchronising call: the next forward, or `check_status`.)
    expect(known_slices <= max_slices_, "slice count exceeds the workspace");
    cur_slices_ = known_slices;
    cur_rows_ = known_rows;
  } else {
    cuda_check(cudaMemcpyAsync(host_header_, plan.data_ptr(), 16 * sizeof(int32_t), cudaMemcpyDeviceToHost, st),
               "plan header copy");
    check_status();  // synchronises the stream: header and status are both on the host now
    expect(host_header_[4] == 0, "routing needs more slices than the workspace was sized for (max_slices)");
    cur_slices_ = host_header_[0];
    cur_rows_ = host_header_[5];
  }
  launch_pass_begin(plan.data_ptr<int>(), lay_, reinterpret_cast<uint32_t*>(expected_total_.data_ptr()),
                    reinterpret_cast<uint32_t*>(pass_base_.data_ptr()),
                    fp8_ ? reinterpret_cast<uint32_t*>(ready_total_.data_ptr()) : nullptr,
                    fp8_ ? reinterpret_cast<uint32_t*>(ready_base_.data_ptr()) : nullptr, st);
  ++launches_;
  ret_target_ += static_cast<uint32_t>(cur_rows_) * static_cast<uint32_t>(D_ / kBlockN);
  if (use_comm_stream_) cuda_check(cudaEventRecord(ev_pass_, st), "event record");
  return cur_slices_;
}

void FusedRank::put(int64_t j, torch::Tensor plan, torch::Tensor order, torch::Tensor x,
                    c10::optional<torch::Tensor> g, torch::Tensor w_flat) {
  expect(j >= 0 && j < cur_slices_, "slice index out of range");
  expect_bf16_2d(x, D_, "x");
  if (g.has_value()) expect_bf16_2d(*g, D_, "g");
  expect(w_flat.is_cuda() && w_flat.scalar_type() == torch::kFloat32 && w_flat.is_contiguous() &&
             w_flat.numel() == cur_rows_,
         "router weights must be a contiguous CUDA fp32 tensor of T*K elements");
  expect_i32(order, cur_rows_, "order");
  cudaStream_t st = use_comm_stream_ ? comm_stream_ : current_stream();
  if (use_comm_stream_) {
    if (j == 0) cuda_check(cudaStreamWaitEvent(comm_stream_, ev_pass_, 0), "wait pass event");
    if (j >= 2) cuda_check(cudaStreamWaitEvent(comm_stream_, ev_done_[(j - 2) % 4], 0), "wait slice event");
  }
  PutParams p{};
  p.plan = plan.data_ptr<int>();
  p.lay = lay_;
  p.slice = static_cast<int>(j);
  p.seq = seq_ + static_cast<uint32_t>(j);
  p.me = me_;
  p.top_k = K_;
  p.hidden = D_;
  p.order = order.data_ptr<int>();
  p.x = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr());
  p.g = g.has_value() ? reinterpret_cast<const __nv_bfloat16*>(g->data_ptr()) : nullptr;
  p.w_flat = w_flat.data_ptr<float>();
  p.num_tokens = static_cast<int>(x.size(0));
  p.peer_x = table<__nv_bfloat16>(kTabX);
  p.peer_g = table<__nv_bfloat16>(kTabG);
  p.peer_w = table<float>(kTabW);
  p.peer_arrive = table<uint32_t>(kTabArrive);
  p.credit = reinterpret_cast<const uint32_t*>(arena_ + arena_lay_.credit);
  p.spin_limit = spin_limit_;
  p.status = reinterpret_cast<StatusBlock*>(status_.data_ptr());
  if (fp8_) {
    p.peer_xq = table<uint8_t>(kTabXq);
    p.peer_gq = table<uint8_t>(kTabGq);
    p.peer_xs = table<float>(kTabXs);
    p.peer_gs = table<float>(kTabGs);
  }
  launch_dispatch_put(p, put_blocks_, st);
  ++launches_;
  if (use_comm_stream_) cuda_check(cudaEventRecord(ev_put_[j % 4], comm_stream_), "event record");
  if (fp8_ && use_comm_stream_) {
    // The expansion of slice j is issued together with its put, one slice ahead of the GEMMs: it waits for arrivals
    // expert by expert while slice j-1 computes. It may overwrite the bf16 slice buffer once slice j-2 is done with it.
    if (j == 0) cuda_check(cudaStreamWaitEvent(expand_stream_, ev_pass_, 0), "wait pass event");
    if (j >= 2) cuda_check(cudaStreamWaitEvent(expand_stream_, ev_done_[(j - 2) % 4], 0), "wait slice event");
    dequant(plan.data_ptr<int>(), static_cast<int>(j), static_cast<int>(p.seq & 1u), g.has_value(), expand_stream_);
    cuda_check(cudaEventRecord(ev_expand_[j % 4], expand_stream_), "event record");
  }
}

GemmParams FusedRank::base_params(const int* plan, int j) const {
  GemmParams p{};
  p.plan = plan;
  p.lay = lay_;
  p.slice = j;
  p.me = me_;
  p.stripe = stripe_;
  p.spin_limit = spin_limit_;
  p.mbar_limit = mbar_limit_;
  p.status = reinterpret_cast<StatusBlock*>(status_.data_ptr());
  return p;
}

const CUtensorMap& FusedRank::weight_map(const torch::Tensor& w, uint32_t box_rows, uint32_t chunks) {
  // Keyed by address AND geometry: a freed tensor's address can come back with another shape.
  auto key = std::make_tuple(static_cast<const void*>(w.data_ptr()), box_rows | (chunks << 16),
                             static_cast<int64_t>(w.size(0)) * w.size(1), static_cast<int64_t>(w.size(2)));
  auto it = weight_maps_.find(key);
  if (it == weight_maps_.end()) {
    if (weight_maps_.size() > 4096) weight_maps_.clear();
    // [L, R, C] viewed as the 2-D matrix [L*R, C]; tiles never straddle experts because R % box_rows == 0.
    const uint64_t rows = static_cast<uint64_t>(w.size(0)) * w.size(1), cols = static_cast<uint64_t>(w.size(2));
    it = weight_maps_.emplace(key, chunks ? make_bf16_map_chunked(w.data_ptr(), rows, cols, box_rows, chunks)
                                          : make_bf16_map_2d(w.data_ptr(), rows, cols, box_rows)).first;
  }
  return it->second;
}

void FusedRank::dequant(const int* plan, int j, int b, bool with_g, cudaStream_t st) {
  // Rows arrived as e4m3 + block scales: expand them into the bf16 slice buffers the GEMMs read.
  DequantParams d{};
  d.plan = plan;
  d.lay = lay_;
  d.slice = j;
  d.hidden = D_;
  d.arrive = reinterpret_cast<const uint32_t*>(arena_ + arena_lay_.arrive);
  d.pass_base = reinterpret_cast<const uint32_t*>(pass_base_.data_ptr());
  const size_t rows_off = static_cast<size_t>(b) * S_;
  d.xq = arena_ + arena_lay_.xq + rows_off * D_;
  d.xs = reinterpret_cast<const float*>(arena_ + arena_lay_.xs) + rows_off * (D_ / 128);
  d.x = reinterpret_cast<__nv_bfloat16*>(arena_ + arena_lay_.xbuf) + rows_off * D_;
  if (with_g) {
    d.gq = arena_ + arena_lay_.gq + rows_off * D_;
    d.gs = reinterpret_cast<const float*>(arena_ + arena_lay_.gs) + rows_off * (D_ / 128);
    d.g = reinterpret_cast<__nv_bfloat16*>(arena_ + arena_lay_.gbuf) + rows_off * D_;
  }
  d.ready = reinterpret_cast<uint32_t*>(ready_.data_ptr());
  d.spin_limit = spin_limit_;
  d.status = reinterpret_cast<StatusBlock*>(status_.data_ptr());
  launch_dequant_slice(d, st);
  ++launches_;
}

void FusedRank::set_pipeline_counters(c10::optional<torch::Tensor> counters) {
  if (!counters.has_value()) {
    prof_ = torch::Tensor();
    return;
  }
  const torch::Tensor& t = *counters;
  expect(t.is_cuda() && t.scalar_type() == torch::kInt64 && t.is_contiguous() && t.dim() == 3 && t.size(0) == 6 &&
             t.size(1) >= num_sms_ && t.size(2) == kProfSlots,
         "pipeline counters must be a contiguous CUDA int64 [6, >= num_sms, 8] tensor");
  prof_ = t;
}

void FusedRank::launch_gemm(int mode, const GemmParams& p0, const CUtensorMap& a, const CUtensorMap& b,
                            cudaStream_t st, const CUtensorMap* c, int spare_sms) {
  GemmParams p = p0;
  if (prof_.defined())
    p.prof = reinterpret_cast<unsigned long long*>(prof_.data_ptr<int64_t>()) +
             static_cast<size_t>(mode) * prof_.size(1) * kProfSlots;
  const CUtensorMap& out = c != nullptr ? *c : a;
  const int grid = std::max(2, num_sms_ - spare_sms);
  if (mode == kModeTgmm ? tgmm_pairs_ : cta_pairs_) launch_grouped_gemm_pair(mode, p, a, b, out, grid, st);
  else launch_grouped_gemm(mode, p, a, b, out, grid, st);
  ++launches_;
}

namespace {
void expect_weights(const torch::Tensor& w_up, const torch::Tensor& w_down, int L, int D, int F) {
  expect(w_up.is_cuda() && w_up.scalar_type() == torch::kBFloat16 && w_up.is_contiguous() && w_up.dim() == 3 &&
             w_up.size(0) == L && w_up.size(1) == D && w_up.size(2) == 2 * F,
         "w_up must be a contiguous CUDA bf16 [L, D, 2F] tensor");
  expect(w_down.is_cuda() && w_down.scalar_type() == torch::kBFloat16 && w_down.is_contiguous() && w_down.dim() == 3 &&
             w_down.size(0) == L && w_down.size(1) == F && w_down.size(2) == D,
         "w_down must be a contiguous CUDA bf16 [L, F, D] tensor");
}
}  // namespace

// Two slices are in flight at a time. Even and odd slices run their kernel chains on two streams with their own
// scratch buffers, the weight-gradient GEMMs and the in-order credit release run on an auxiliary stream, the puts on
// the comm stream. A persistent GEMM kernel needs a whole SM per CTA, so two ready kernels do not share SMs: the
// later one's CTAs start as the earlier one's CTAs finish, i.e. every kernel fills the idle tail of the previous
// (independent) one instead of waiting for it. Scratch reuse and the carry chain are ordered by events.
void FusedRank::compute_forward(int64_t j, torch::Tensor plan, torch::Tensor w_up, torch::Tensor w_down) {
  expect(j >= 0 && j < cur_slices_, "slice index out of range");
  expect_weights(w_up, w_down, L_, D_, F_);
  const bool async = use_comm_stream_;
  const int q = static_cast<int>(j & 1);
  cudaStream_t st = async ? chain_[q] : current_stream();
  cudaStream_t aux = async ? aux_stream_ : st;
  if (async) {
    if (j < 2) cuda_check(cudaStreamWaitEvent(st, ev_pass_, 0), "wait pass event");
    cuda_check(cudaStreamWaitEvent(st, ev_put_[j % 4], 0), "wait put event");
  }
  const uint32_t seq = seq_ + static_cast<uint32_t>(j);
  const int b = static_cast<int>(seq & 1u);
  const int* pl = plan.data_ptr<int>();
  if (fp8_ && !async) dequant(pl, static_cast<int>(j), b, /*with_g=*/false, st);  // lockstep: every put is done
  {
    GemmParams p = base_params(pl, static_cast<int>(j));
    p.n_tiles = 2 * F_ / kBlockN;
    p.k_blocks = D_ / kBlockK;
    p.b_group_rows = D_;
    p.arrive = fp8_ ? nullptr : reinterpret_cast<const uint32_t*>(arena_ + arena_lay_.arrive);
    p.pass_base = reinterpret_cast<const uint32_t*>(pass_base_.data_ptr());
    p.ready = fp8_ ? reinterpret_cast<const uint32_t*>(ready_.data_ptr()) : nullptr;
    p.ready_base = reinterpret_cast<const uint32_t*>(ready_base_.data_ptr());
    p.out0 = reinterpret_cast<__nv_bfloat16*>(act_[q].data_ptr());
    p.ld0 = F_;
    p.out1 = nullptr;
    p.ld1 = 2 * F_;
    // fp8 wire: this kernel waits (in its producer warp) for the expansion kernel of the same slice. A persistent CTA
    // takes all of an SM's shared memory, so nothing else can start beside it: the kernel leaves a few SMs free for the
    // expansion kernel, and it only starts once the expansion of the PREVIOUS slice has finished, so that at most one
    // kernel is ever waiting for an expansion that still needs SMs.
    if (fp8_ && async && j >= 1) cuda_check(cudaStreamWaitEvent(st, ev_expand_[(j - 1) % 4], 0), "wait expansion");
    launch_gemm(kModeSwiglu, p, map_x_k_[b], weight_map(w_up, 64, cta_pairs_ ? 2 : 4), st, nullptr,
                fp8_ && async ? kExpandSms : 0);
  }
  {
    GemmParams p = base_params(pl, static_cast<int>(j));
    p.n_tiles = D_ / kBlockN;
    p.k_blocks = F_ / kBlockK;
    p.b_group_rows = F_;
    p.row_w = reinterpret_cast<const float*>(arena_ + arena_lay_.wbuf) + static_cast<size_t>(b) * S_;
    p.peer_rows = table<__nv_bfloat16>(kTabRet);
    p.ret_blocked = ret_blocked_ ? 1 : 0;
    p.ret_lsu = ret_lsu_ ? 1 : 0;
    p.ret_rows = tk_cap_;
    p.peer_count = table<uint32_t>(kTabCount);
    p.ld0 = D_;
    launch_gemm(kModeDownFwd, p, map_act_k_[q], weight_map(w_down, 64, cta_pairs_ ? 2 : 4), st);
  }
  if (async) {
    cuda_check(cudaEventRecord(ev_down_[q], st), "event record");
    cuda_check(cudaStreamWaitEvent(aux, ev_down_[q], 0), "wait down event");
  }
  launch_slice_done(table<uint32_t>(kTabCredit), P_, me_, seq, aux);  // credits leave in slice order
  ++launches_;
  if (async) cuda_check(cudaEventRecord(ev_done_[j % 4], aux), "event record");
}

void FusedRank::compute_backward(int64_t j, torch::Tensor plan, torch::Tensor w_up, torch::Tensor w_down,
                                 torch::Tensor dw_up, torch::Tensor dw_down) {
  expect(j >= 0 && j < cur_slices_, "slice index out of range");
  expect_weights(w_up, w_down, L_, D_, F_);
  expect_weights(dw_up, dw_down, L_, D_, F_);
  const bool async = use_comm_stream_;
  const int q = static_cast<int>(j & 1);
  cudaStream_t st = async ? chain_[q] : current_stream();
  cudaStream_t aux = async ? aux_stream_ : st;
  if (async) {
    if (j < 2) cuda_check(cudaStreamWaitEvent(st, ev_pass_, 0), "wait pass event");
    cuda_check(cudaStreamWaitEvent(st, ev_put_[j % 4], 0), "wait put event");
    if (j >= 2) cuda_check(cudaStreamWaitEvent(st, ev_tgd_[q], 0), "wait dW_down event");  // act, h, dy of slice j-2
  }
  const uint32_t seq = seq_ + static_cast<uint32_t>(j);
  const int b = static_cast<int>(seq & 1u);
  const int* pl = plan.data_ptr<int>();
  const int par = static_cast<int>(j & 1);
  const int dwp_tiles = D_ / kBlockN;
  if (fp8_ && !async) dequant(pl, static_cast<int>(j), b, /*with_g=*/true, st);  // lockstep: every put is done
  {  // remat: act and h
    GemmParams p = base_params(pl, static_cast<int>(j));
    p.n_tiles = 2 * F_ / kBlockN;
    p.k_blocks = D_ / kBlockK;
    p.b_group_rows = D_;
    p.arrive = fp8_ ? nullptr : reinterpret_cast<const uint32_t*>(arena_ + arena_lay_.arrive);
    p.pass_base = reinterpret_cast<const uint32_t*>(pass_base_.data_ptr());
    p.ready = fp8_ ? reinterpret_cast<const uint32_t*>(ready_.data_ptr()) : nullptr;
    p.ready_base = reinterpret_cast<const uint32_t*>(ready_base_.data_ptr());
    p.out0 = reinterpret_cast<__nv_bfloat16*>(act_[q].data_ptr());
    p.ld0 = F_;
    p.out1 = reinterpret_cast<__nv_bfloat16*>(h_[q].data_ptr());
    p.ld1 = 2 * F_;
    // fp8 wire: this kernel waits (in its producer warp) for the expansion kernel of the same slice. A persistent CTA
    // takes all of an SM's shared memory, so nothing else can start beside it: the kernel leaves a few SMs free for the
    // expansion kernel, and it only starts once the expansion of the PREVIOUS slice has finished, so that at most one
    // kernel is ever waiting for an expansion that still needs SMs.
    if (fp8_ && async && j >= 1) cuda_check(cudaStreamWaitEvent(st, ev_expand_[(j - 1) % 4], 0), "wait expansion");
    launch_gemm(kModeSwiglu, p, map_x_k_[b], weight_map(w_up, 64, cta_pairs_ ? 2 : 4), st, nullptr,
                fp8_ && async ? kExpandSms : 0);
  }
  {  // remat of y, folded into d_weight partials; dy = w * g
    GemmParams p = base_params(pl, static_cast<int>(j));
    p.n_tiles = D_ / kBlockN;
    p.k_blocks = F_ / kBlockK;
    p.b_group_rows = F_;
    p.row_w = reinterpret_cast<const float*>(arena_ + arena_lay_.wbuf) + static_cast<size_t>(b) * S_;
    p.in0 = reinterpret_cast<const __nv_bfloat16*>(arena_ + arena_lay_.gbuf) + static_cast<size_t>(b) * S_ * D_;
    p.out0 = reinterpret_cast<__nv_bfloat16*>(dy_[q].data_ptr());
    p.ld0 = D_;
    p.dwp = dwp_[q].data_ptr<float>();
    p.dwp_tiles = dwp_tiles;
    launch_gemm(kModeDownDw, p, map_act_k_[q], weight_map(w_down, 64, cta_pairs_ ? 2 : 4), st);
  }
  if (async) {
    cuda_check(cudaEventRecord(ev_dd_[q], st), "event record");
    if (j >= 2) cuda_check(cudaStreamWaitEvent(st, ev_tgu_[q], 0), "wait dW_up event");  // dh of slice j-2
  }
  {  // dh = SwiGLU'(h) * (dy Wd^T)
    GemmParams p = base_params(pl, static_cast<int>(j));
    p.n_tiles = F_ / kBlockN;
    p.k_blocks = D_ / kBlockK;
    p.b_group_rows = F_;
    p.in0 = reinterpret_cast<const __nv_bfloat16*>(h_[q].data_ptr());
    p.out0 = reinterpret_cast<__nv_bfloat16*>(dh_[q].data_ptr());
    p.ld0 = 2 * F_;
    launch_gemm(kModeDswiglu, p, map_dy_k_[q], weight_map(w_down, cta_pairs_ ? 128 : 256), st);
  }
  if (async) {
    cuda_check(cudaEventRecord(ev_ds_[q], st), "event record");
    cuda_check(cudaStreamWaitEvent(aux, ev_dd_[q], 0), "wait down event");
  }
  {  // dW_down[g] = act^T dy   (auxiliary stream; the fp32 carry chains slice to slice there)
    GemmParams p = base_params(pl, static_cast<int>(j));
    p.m_tiles = F_ / kBlockM;
    p.n_tiles = D_ / kBlockN;
    p.carry_in = carry_down_.data_ptr<float>() + static_cast<size_t>(par ^ 1) * F_ * D_;
    p.carry_out = carry_down_.data_ptr<float>() + static_cast<size_t>(par) * F_ * D_;
    p.grad_out = reinterpret_cast<__nv_bfloat16*>(dw_down.data_ptr());
    launch_gemm(kModeTgmm, p, map_act_mn_[q], map_dy_mn_[q], aux, &weight_map(dw_down, 32));
  }
  if (async) {
    cuda_check(cudaEventRecord(ev_tgd_[q], aux), "event record");
    cuda_check(cudaStreamWaitEvent(aux, ev_ds_[q], 0), "wait dswiglu event");
  }
  {  // dx = dh Wu^T, rows and d_weight go back to their source rank
    GemmParams p = base_params(pl, static_cast<int>(j));
    p.n_tiles = D_ / kBlockN;
    p.k_blocks = 2 * F_ / kBlockK;
    p.b_group_rows = D_;
    p.peer_rows = table<__nv_bfloat16>(kTabRet);
    p.ret_blocked = ret_blocked_ ? 1 : 0;
    p.ret_lsu = ret_lsu_ ? 1 : 0;
    p.ret_rows = tk_cap_;
    p.peer_dw = table<float>(kTabDw);
    p.peer_count = table<uint32_t>(kTabCount);
    p.ld0 = D_;
    p.dwp = dwp_[q].data_ptr<float>();
    p.dwp_tiles = dwp_tiles;
    launch_gemm(kModeDx, p, map_dh_k_[q], weight_map(w_up, cta_pairs_ ? 128 : 256), st);
  }
  if (async) cuda_check(cudaEventRecord(ev_dx_[q], st), "event record");
  {  // dW_up[g] = x^T dh
    GemmParams p = base_params(pl, static_cast<int>(j));
    p.m_tiles = D_ / kBlockM;
    p.n_tiles = 2 * F_ / kBlockN;
    p.carry_in = carry_up_.data_ptr<float>() + static_cast<size_t>(par ^ 1) * D_ * 2 * F_;
    p.carry_out = carry_up_.data_ptr<float>() + static_cast<size_t>(par) * D_ * 2 * F_;
    p.grad_out = reinterpret_cast<__nv_bfloat16*>(dw_up.data_ptr());
    launch_gemm(kModeTgmm, p, map_x_mn_[b], map_dh_mn_[q], aux, &weight_map(dw_up, 32));
  }
  if (async) cuda_check(cudaEventRecord(ev_tgu_[q], aux), "event record");
  launch_slice_done(table<uint32_t>(kTabCredit), P_, me_, seq, aux);
  ++launches_;
  if (async) cuda_check(cudaEventRecord(ev_done_[j % 4], aux), "event record");
}

// Makes the caller's stream wait for everything the pass issued on the chain and auxiliary streams.
void FusedRank::join_streams(bool backward) {
  if (!use_comm_stream_ || cur_slices_ <= 0) return;
  cudaStream_t st = current_stream();
  cuda_check(cudaStreamWaitEvent(st, ev_done_[(cur_slices_ - 1) % 4], 0), "join aux stream");
  if (fp8_) cuda_check(cudaStreamWaitEvent(st, ev_expand_[(cur_slices_ - 1) % 4], 0), "join expand stream");
  if (backward) {
    cuda_check(cudaStreamWaitEvent(st, ev_dx_[(cur_slices_ - 1) & 1], 0), "join chain stream");
    if (cur_slices_ >= 2) cuda_check(cudaStreamWaitEvent(st, ev_dx_[cur_slices_ & 1], 0), "join chain stream");
  }
}

void FusedRank::end_pass(int64_t n_slices) {
  seq_ += static_cast<uint32_t>(n_slices);
  cur_slices_ = 0;
}

void FusedRank::finish_forward(torch::Tensor inv_order, torch::Tensor out) {
  expect_bf16_2d(out, D_, "out");
  expect(out.size(0) * K_ == cur_rows_, "out rows do not match the pass");
  expect_i32(inv_order, cur_rows_, "inv_order");
  join_streams(/*backward=*/false);
  CombineParams c{};
  c.rows = reinterpret_cast<const __nv_bfloat16*>(arena_ + arena_lay_.ret);
  c.inv_order = inv_order.data_ptr<int>();
  c.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  c.num_tokens = static_cast<int>(out.size(0));
  c.top_k = K_;
  c.hidden = D_;
  c.blocked = ret_blocked_ ? 1 : 0;
  c.ret_rows = tk_cap_;
  c.count = reinterpret_cast<const uint32_t*>(arena_ + arena_lay_.ret_count);
  c.target = ret_target_;
  c.spin_limit = spin_limit_;
  c.status = reinterpret_cast<StatusBlock*>(status_.data_ptr());
  launch_combine_reduce(c, current_stream());
  ++launches_;
  end_pass(cur_slices_);
}

void FusedRank::finish_backward(torch::Tensor inv_order, torch::Tensor dx, torch::Tensor d_weights) {
  expect_bf16_2d(dx, D_, "dx");
  expect(dx.size(0) * K_ == cur_rows_, "dx rows do not match the pass");
  expect(d_weights.is_cuda() && d_weights.scalar_type() == torch::kFloat32 && d_weights.is_contiguous() &&
             d_weights.numel() == cur_rows_,
         "d_weights must be a contiguous CUDA fp32 tensor of T*K elements");
  expect_i32(inv_order, cur_rows_, "inv_order");
  join_streams(/*backward=*/true);
  CombineParams c{};
  c.rows = reinterpret_cast<const __nv_bfloat16*>(arena_ + arena_lay_.ret);
  c.inv_order = inv_order.data_ptr<int>();
  c.out = reinterpret_cast<__nv_bfloat16*>(dx.data_ptr());
  c.dw_rows = reinterpret_cast<const float*>(arena_ + arena_lay_.dw_rows);
  c.d_weights = d_weights.data_ptr<float>();
  c.num_tokens = static_cast<int>(dx.size(0));
  c.top_k = K_;
  c.hidden = D_;
  c.blocked = ret_blocked_ ? 1 : 0;
  c.ret_rows = tk_cap_;
  c.count = reinterpret_cast<const uint32_t*>(arena_ + arena_lay_.ret_count);
  c.target = ret_target_;
  c.spin_limit = spin_limit_;
  c.status = reinterpret_cast<StatusBlock*>(status_.data_ptr());
  launch_combine_reduce(c, current_stream());
  ++launches_;
  end_pass(cur_slices_);
}

// ---------------------------------------------------------------------------------------------
// symmetric arena: cudaMalloc + CUDA IPC handles
// ---------------------------------------------------------------------------------------------
int64_t arena_alloc(int64_t bytes) {
  void* p = nullptr;
  cuda_check(cudaMalloc(&p, static_cast<size_t>(bytes)), "arena cudaMalloc");
  cuda_check(cudaMemset(p, 0, static_cast<size_t>(bytes)), "arena memset");
  cuda_check(cudaDeviceSynchronize(), "arena sync");
  return reinterpret_cast<int64_t>(p);
}

void arena_free(int64_t ptr) { cudaFree(reinterpret_cast<void*>(ptr)); }

py::bytes arena_export(int64_t ptr) {
  cudaIpcMemHandle_t h;
  cuda_check(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(ptr)), "cudaIpcGetMemHandle");
  return py::bytes(reinterpret_cast<const char*>(&h), sizeof(h));
}

int64_t arena_import(py::bytes handle) {
  std::string s = handle;
  expect(s.size() == sizeof(cudaIpcMemHandle_t), "bad IPC handle size");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, s.data(), sizeof(h));
  void* p = nullptr;
  cuda_check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return reinterpret_cast<int64_t>(p);
}

void arena_close(int64_t ptr) { cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)); }

void arena_zero(int64_t ptr, int64_t bytes) {
  cuda_check(cudaMemset(reinterpret_cast<void*>(ptr), 0, static_cast<size_t>(bytes)), "arena memset");
  cuda_check(cudaDeviceSynchronize(), "arena sync");
}

torch::Tensor arena_read_i32(int64_t ptr, int64_t offset_bytes, int64_t count) {
  expect(ptr != 0 && offset_bytes >= 0 && offset_bytes % 4 == 0 && count >= 0, "bad arena range");
  torch::Tensor out = torch::empty({count}, torch::kInt32);
  cuda_check(cudaDeviceSynchronize(), "arena sync");
  cuda_check(cudaMemcpy(out.data_ptr(), reinterpret_cast<const uint8_t*>(ptr) + offset_bytes,
                        static_cast<size_t>(count) * 4, cudaMemcpyDeviceToHost),
             "arena read");
  return out;
}

void arena_fill(int64_t ptr, int64_t bytes, int value) {
  cuda_check(cudaMemset(reinterpret_cast<void*>(ptr), value, static_cast<size_t>(bytes)), "arena memset");
  cuda_check(cudaDeviceSynchronize(), "arena sync");
}

}  // namespace cem
