// Per-rank executor of the fused NVLink path: owns the scratch buffers, the peer pointer tables,
// the TMA descriptors, the comm stream and the slice sequence counter, and launches the kernels
// of one slice at a time.
//
// The step methods (begin_*, put, compute_*, finish_*) are what a pass is made of:
//
//     begin_forward -> put(0) -> for j: put(j+1); compute_forward(j) -> finish_forward
//
// One process drives one rank per GPU that way. A test harness may instead drive several
// ranks that live on ONE device in lockstep (all puts of a slice, then all computes); then
// every flag a kernel looks at has already been set when it starts and nothing ever spins.
#pragma once

#include <torch/extension.h>

#include <cuda.h>
#include <cuda_runtime.h>

#include <map>
#include <string>
#include <tuple>
#include <vector>

#include "../comm/comm_kernels.cuh"
#include "../gemm/grouped_gemm.cuh"
#include "../plan/plan_kernel.cuh"

namespace cem {

// Byte offsets inside one rank's symmetric arena (identical on every rank).
struct ArenaLayout {
  size_t xbuf, gbuf, wbuf, xq, gq, xs, gs, ret, dw_rows, arrive, credit, ret_count, traffic, traffic_flags, total;
};

ArenaLayout make_arena_layout(int P, int L, int S, int D, int tk_cap, bool fp8);

// Text of a recorded status block {code, kernel, mode, slice, detail, expected, seen, block} (what check_status raises).
std::string format_status(const std::vector<int64_t>& status, int rank);

class FusedRank {
 public:
  FusedRank(int P, int L, int me, int S, int D, int F, int K, int stripe, int tk_cap, int max_slices, int num_sms,
            bool fp8, int64_t arena, std::vector<int64_t> peer_arenas, bool use_comm_stream, int64_t spin_limit,
            int put_blocks, bool cta_pairs, bool tgmm_pairs);
  ~FusedRank();

  // Forward pass set-up: sort, traffic exchange, plan tables, arrival targets. `plan`, `order`,
  // `inv_order` are caller-owned int32 tensors (they are what the backward needs again).
  // With `counts_prefilled` the [P,P,L] traffic matrix in `counts` is taken as is (lockstep harness).
  // Returns the number of slices (this synchronises the host with the plan kernel once).
  int64_t begin_forward(torch::Tensor expert_ids, torch::Tensor plan, torch::Tensor order, torch::Tensor inv_order,
                        torch::Tensor counts, bool counts_prefilled);
  // The same set-up without waiting for the device: the plan header and the status block are copied to pinned host
  // memory behind the plan kernel and an event is recorded. Returns the slice count of this workspace's previous
  // forward pass (-1 if there was none) as a GUESS; the caller may launch that many slices at once, then calls
  // `resolve_slices()` for the real count, launches what is still missing and reports what it launched with
  // `set_pass_slices()`. Slices past the real count find empty tables and do nothing, on every rank alike.
  int64_t begin_forward_async(torch::Tensor expert_ids, torch::Tensor plan, torch::Tensor order,
                              torch::Tensor inv_order, torch::Tensor counts, bool counts_prefilled);
  // Waits for the header copy (not for the stream), raises a recorded kernel error, returns the real slice count.
  int64_t resolve_slices();
  void set_pass_slices(int64_t launched);
  // Microseconds a pipeline barrier inside a GEMM may take before the kernel gives up (default 20 s).
  void set_mbar_limit_us(int64_t us);
  // Lockstep harness only: sort + histogram without the exchange (fills order, inv_order, my row of counts).
  void sort_only(torch::Tensor expert_ids, torch::Tensor order, torch::Tensor inv_order, torch::Tensor my_counts);
  // `known_slices`, `known_rows` (T*K): what the forward of the same plan returned / was given; when both are >= 0
  // the plan header is not read back and the stream is not synchronised.
  int64_t begin_backward(torch::Tensor plan, int64_t known_slices = -1, int64_t known_rows = -1);

  void put(int64_t j, torch::Tensor plan, torch::Tensor order, torch::Tensor x, c10::optional<torch::Tensor> g,
           torch::Tensor w_flat);
  void compute_forward(int64_t j, torch::Tensor plan, torch::Tensor w_up, torch::Tensor w_down);
  void compute_backward(int64_t j, torch::Tensor plan, torch::Tensor w_up, torch::Tensor w_down, torch::Tensor dw_up,
                        torch::Tensor dw_down);
  void finish_forward(torch::Tensor inv_order, torch::Tensor out);
  void finish_backward(torch::Tensor inv_order, torch::Tensor dx, torch::Tensor d_weights);

  // Reads the status block (synchronises); throws std::runtime_error describing the first recorded error.
  void check_status();
  std::vector<int64_t> plan_header() const { return std::vector<int64_t>(host_header_, host_header_ + 16); }
  int64_t plan_ints() const { return lay_.total; }
  int64_t launches() const { return launches_; }
  // Turns the GEMM kernels' pipeline counters on: `counters` is a zeroed int64 CUDA tensor [6 modes, num_sms, 8]
  // (slots: ProfSlot in gemm/grouped_gemm.cuh) that every later GEMM launch adds to. An undefined tensor turns
  // them off again. Diagnostics only: the counting costs a few clock reads per k-block.
  void set_pipeline_counters(c10::optional<torch::Tensor> counters);
  // Debug views of the local scratch (tests compare them with the torch reference).
  torch::Tensor act() const { return act_[0]; }
  torch::Tensor h() const { return h_[0]; }
  torch::Tensor dh() const { return dh_[0]; }
  torch::Tensor dy() const { return dy_[0]; }

 private:
  void end_pass(int64_t n_slices);
  void join_streams(bool backward);
  GemmParams base_params(const int* plan, int j) const;
  // `chunks` > 0: the MN-major description (64-column chunks, `chunks` of them per copy); 0: plain 2-D boxes.
  const CUtensorMap& weight_map(const torch::Tensor& w, uint32_t box_rows, uint32_t chunks = 0);
  void dequant(const int* plan, int j, int b, bool with_g, cudaStream_t st);
  // `c`: the output's tensor map (weight-gradient mode: tiled stores of the bf16 gradient); null otherwise.
  void launch_gemm(int mode, const GemmParams& p, const CUtensorMap& a, const CUtensorMap& b, cudaStream_t st,
                   const CUtensorMap* c = nullptr, int spare_sms = 0);

  int P_, L_, me_, S_, D_, F_, K_, stripe_, tk_cap_, max_slices_, num_sms_, put_blocks_;
  // `cta_pairs_`: the row-wise GEMM modes run as CTA pairs (256-row tiles). `tgmm_pairs_`: the weight-gradient mode
  // does; its pairs split the dense feature dimension, so they cost no token padding and are on by default.
  bool fp8_, use_comm_stream_, cta_pairs_, tgmm_pairs_;
  bool ret_lsu_ = false;      // CEM_RET_LSU: combine epilogues write staged rows with vector stores, not bulk stores
  bool ret_blocked_ = false;  // CEM_RET_BLOCKED: return buffers kept column tile by column tile (every rank alike)
  uint32_t spin_limit_, mbar_limit_;
  PlanLayout lay_;
  ArenaLayout arena_lay_;
  uint8_t* arena_;
  std::vector<uint8_t*> peers_;

  // local scratch (torch-owned)
  torch::Tensor act_[2], h_[2], dy_[2], dh_[2], dwp_[2];
  torch::Tensor carry_up_, carry_down_, pass_base_, expected_total_, status_, tables_,
      sort_scratch_, my_counts_;
  torch::Tensor ready_, ready_base_, ready_total_;  // fp8 wire: per-expert "rows expanded" counter, its base, its target
  // device pointer tables, rows of `tables_`
  enum Table { kTabX, kTabG, kTabW, kTabXq, kTabGq, kTabXs, kTabGs, kTabArrive, kTabRet, kTabDw, kTabCount,
               kTabCredit, kTabTraffic0, kTabTraffic1, kTabTflags0, kTabTflags1, kNumTables };
  template <typename T>
  T* const* table(int t) const { return reinterpret_cast<T* const*>(tables_.data_ptr<int64_t>() + t * P_); }

  CUtensorMap map_x_k_[2], map_x_mn_[2], map_act_k_[2], map_act_mn_[2], map_dy_k_[2], map_dy_mn_[2], map_dh_k_[2],
      map_dh_mn_[2];
  std::map<std::tuple<const void*, uint32_t, int64_t, int64_t>, CUtensorMap> weight_maps_;

  cudaStream_t comm_stream_ = nullptr, aux_stream_ = nullptr, chain_[2] = {};
  cudaStream_t expand_stream_ = nullptr;  // fp8 wire: the expansion kernels run here, beside the GEMM chains
  cudaEvent_t ev_expand_[4] = {};  // expansion of slice j (mod 4) has finished
  cudaEvent_t ev_down_[2] = {}, ev_dd_[2] = {}, ev_ds_[2] = {}, ev_dx_[2] = {}, ev_tgd_[2] = {}, ev_tgu_[2] = {};
  cudaEvent_t ev_pass_ = nullptr, ev_put_[4] = {}, ev_done_[4] = {}, ev_header_ = nullptr;
  int64_t last_slices_ = -1;  // slice count of the previous forward pass (the next pass's guess)
  int32_t* host_header_ = nullptr;  // pinned: 16 plan header ints + 8 status ints

  uint32_t seq_ = 0;          // global slice sequence number of the next pass's first slice
  uint32_t fwd_epoch_ = 0;    // forward passes started (traffic exchange epoch)
  uint32_t ret_target_ = 0;   // value the returned-row counter reaches at the end of the current pass
  int64_t cur_slices_ = 0;
  int64_t cur_rows_ = 0;      // T*K of the current pass
  int64_t launches_ = 0;
  torch::Tensor prof_;
};

// Symmetric arena helpers (cudaMalloc + CUDA IPC), one arena per rank.
int64_t arena_alloc(int64_t bytes);
void arena_free(int64_t ptr);
py::bytes arena_export(int64_t ptr);
int64_t arena_import(py::bytes handle);
void arena_close(int64_t ptr);
void arena_zero(int64_t ptr, int64_t bytes);
void arena_fill(int64_t ptr, int64_t bytes, int value);
// Synchronises the device and copies `count` int32 values at `ptr + offset_bytes` to a CPU tensor (tests read counters).
torch::Tensor arena_read_i32(int64_t ptr, int64_t offset_bytes, int64_t count);

}  // namespace cem
