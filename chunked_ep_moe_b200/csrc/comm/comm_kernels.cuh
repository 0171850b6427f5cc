// One-sided NVLink dispatch (put + arrival counters), buffer credits and the K-way combine reduce.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/status.cuh"
#include "../plan/plan_tables.cuh"

namespace cem {

struct PutParams {
  const int* plan;
  PlanLayout lay;
  int slice;            // slice index inside the pass
  uint32_t seq;         // global slice sequence number (selects the double buffer, orders credits)
  int me, top_k, hidden;
  int num_tokens;       // rows of x (and g): send-order entries are checked against it
  const int* order;                 // [T*K] flat assignment index t*K+k at each send-order position
  const __nv_bfloat16* x;           // [T, D] tokens (gathered by token id: no send-order copy exists)
  const __nv_bfloat16* g;           // [T, D] output gradient, or null in the forward
  const float* w_flat;              // [T*K] router weights
  __nv_bfloat16* const* peer_x;     // [P] each receiver's x slice buffers  [2][S][D]
  __nv_bfloat16* const* peer_g;     // [P] each receiver's g slice buffers  [2][S][D]
  float* const* peer_w;             // [P] each receiver's router-weight slice buffers [2][S]
  uint32_t* const* peer_arrive;     // [P] each receiver's arrival counters [P*L], index source*L + expert
  const uint32_t* credit;           // [P] local: slices receiver r has finished with (written by r)
  uint32_t spin_limit;
  StatusBlock* status;
  // fp8 wire (comm_dtype=float8_e4m3fn): rows travel as e4m3 + one fp32 scale per 128 columns
  uint8_t* const* peer_xq;          // [P] [2][S][D] e4m3, or null when rows travel in bf16
  uint8_t* const* peer_gq;
  float* const* peer_xs;            // [P] [2][S][D/128] scales
  float* const* peer_gs;
};

void launch_dispatch_put(const PutParams& p, int grid, cudaStream_t stream);

// Tells every sender that this rank has finished reading the slice buffers of sequence `seq`.
void launch_slice_done(uint32_t* const* peer_credit, int num_ranks, int me, uint32_t seq, cudaStream_t stream);

// Snapshot of the counter targets at the start of a pass: base = total; total += rows expected. `expected_total` /
// `pass_base` are the [P*L] arrival counters' totals and bases; `ready_total` / `ready_base` ([L], may be null) the
// same for the per-expert "rows expanded" counters of the fp8 wire.
void launch_pass_begin(const int* plan, PlanLayout lay, uint32_t* expected_total, uint32_t* pass_base,
                       uint32_t* ready_total, uint32_t* ready_base, cudaStream_t stream);

struct CombineParams {
  const __nv_bfloat16* rows;  // [T*K, D] returned rows in send order
  const int* inv_order;       // [T*K] send-order position of flat assignment t*K+k
  __nv_bfloat16* out;         // [T, D]
  const float* dw_rows;       // [T*K] returned d_weight rows (backward) or null
  float* d_weights;           // [T*K] flat by t*K+k (backward) or null
  int num_tokens, top_k, hidden;
  int blocked, ret_rows;      // `rows` is kept column tile by column tile: [hidden/256][ret_rows][256], 16-byte pieces
                              // of a row piece XOR-ed with the low three bits of the row number
  const uint32_t* count;      // returned-row counter on this rank
  uint32_t target;            // value the counter reaches when everything is back
  uint32_t spin_limit;
  StatusBlock* status;
};

void launch_combine_reduce(const CombineParams& p, cudaStream_t stream);

// Receiver-side expansion of arrived fp8 rows (e4m3 + one fp32 scale per 128 columns) into the bf16 slice buffer
// the GEMMs read, expert by expert: the kernel acquires the arrival counters of ONE expert's segments, expands that
// expert's rows, releases the row count to the expert's `ready` counter, and goes on to the next expert. The
// up-projection GEMM's producer waits on `ready`, so expansion and transfer of later experts overlap the tiles of
// earlier ones, as arrival does on the bf16 wire.
struct DequantParams {
  const int* plan;
  PlanLayout lay;
  int slice;
  int hidden;
  const uint32_t* arrive;
  const uint32_t* pass_base;
  const uint8_t* xq;          // [S, D] e4m3
  const float* xs;            // [S, D/128]
  __nv_bfloat16* x;           // [S, D]
  const uint8_t* gq;          // backward: the output gradient's slice, or null
  const float* gs;
  __nv_bfloat16* g;
  uint32_t* ready;            // [L] cumulative rows of local expert l expanded so far (local counter, only grows)
  uint32_t spin_limit;
  StatusBlock* status;
};

void launch_dequant_slice(const DequantParams& p, cudaStream_t stream);

// Bounded-wait self test: waits on a counter nobody advances and reports through `status`.
void launch_wait_probe(const uint32_t* flag, uint32_t target, uint32_t spin_limit, StatusBlock* status,
                       cudaStream_t stream);

}  // namespace cem
