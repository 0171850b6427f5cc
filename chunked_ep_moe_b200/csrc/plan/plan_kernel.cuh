// Device-side plan construction: traffic-matrix exchange over NVLink + table build in one kernel,
// and the stable counting sort of token copies by expert.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/status.cuh"
#include "plan_tables.cuh"

namespace cem {

struct PlanKernelParams {
  PlanLayout lay;
  int me;
  const int* my_counts;            // [P*L] this rank's histogram (global expert order = receiver-major)
  int* counts;                     // [P*P*L] this rank's copy of the traffic matrix for this parity
  int* const* peer_counts;         // [P] every rank's traffic buffer for this parity (null when P == 1 and local)
  uint32_t* const* peer_flags;     // [P] every rank's [P] "row s has landed" epoch flags for this parity
  const uint32_t* flags;           // this rank's flags for this parity
  uint32_t epoch;                  // forward-pass counter; flags reach it when a row has landed
  int* plan;                       // output tables
  uint32_t spin_limit;
  StatusBlock* status;
  int use_smem = 0;                // set by the launcher: the tables are built from a shared-memory copy of the matrix
};

// Exchanges the [P, L] histograms (each rank stores its row into every peer and releases a flag),
// waits for all rows, then builds the per-pass tables. Replaces the reference's all_gather +
// prefix sums + per-slice argument builders (src/chunked_moe/plan.py:77-163).
void launch_plan_build(const PlanKernelParams& p, cudaStream_t stream);

// Host restatement of the table build, for CPU tests of the shared arithmetic.
void plan_build_host(const int* counts, int* plan, const PlanLayout& lay, int me);

// Stable counting sort of the T*K expert ids: order (send order -> flat index), inverse, histogram.
// Replaces argsort + scatter-add bincount (src/chunked_moe/plan.py:74-76). Ids outside [0, num_experts) take no part
// in the sort (their `inv_order` entry and the tail of `order` are left untouched); with a status block the first one
// is recorded as kStatusBadIndex (detail = its position, expected = num_experts, seen = the id).
void launch_expert_sort(const int* expert_ids, int n, int num_experts, int* order, int* inv_order, int* counts,
                        int* scratch, cudaStream_t stream, StatusBlock* status = nullptr);
size_t expert_sort_scratch_ints(int n, int num_experts);

}  // namespace cem
