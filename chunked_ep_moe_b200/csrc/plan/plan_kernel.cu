// Plan kernel (single CTA) and expert sort.
#include "plan_kernel.cuh"

#include "../common/umma.cuh"

namespace cem {

namespace {

__global__ void __launch_bounds__(256) plan_build_kernel(const PlanKernelParams p) {
  __shared__ int s_abort;
  const int P = p.lay.P, n = P * p.lay.L;
  if (threadIdx.x == 0) s_abort = 0;
  // 1. publish my histogram row into every rank's traffic matrix (row index = me)
  for (int r = 0; r < P; ++r) {
    int* dst = (p.peer_counts != nullptr ? p.peer_counts[r] : p.counts) + p.me * n;
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = p.my_counts[i];
  }
  __syncthreads();
  if (p.peer_flags != nullptr) {
    if (threadIdx.x < P) {
      __threadfence_system();
      st_release_sys(p.peer_flags[threadIdx.x] + p.me, p.epoch);
    }
    // 2. wait for every rank's row to land here
    if (threadIdx.x < P) {
      uint32_t seen = 0;
      if (!spin_until_reached(p.flags + threadIdx.x, p.epoch, p.spin_limit, &seen)) {
        report_status(p.status, kStatusTrafficTimeout, kKernelPlan, 0, static_cast<int>(p.epoch), threadIdx.x, p.epoch, seen);
        s_abort = 1;
      }
    }
  }
  __syncthreads();
  if (s_abort) {
    if (threadIdx.x == 0) p.plan[0] = 0;  // zero slices: the pass launches nothing
    return;
  }
  // 3. tables
  plan_phase_a(p.counts, p.plan, p.lay, p.me, threadIdx.x, blockDim.x);
  __syncthreads();
  plan_phase_b(p.plan, p.lay, threadIdx.x, blockDim.x);
}

// ---- expert sort: per-block histograms -> exclusive scan over (expert, block) -> stable scatter ----
constexpr int kSortThreads = 256;
constexpr int kSortItems = 8;  // ids per thread; one block covers 2048 consecutive ids

__global__ void __launch_bounds__(kSortThreads) sort_hist_kernel(const int* ids, int n, int num_experts, int* block_hist,
                                                                  StatusBlock* status) {
  extern __shared__ int s_hist[];
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) s_hist[e] = 0;
  __syncthreads();
  const int base = blockIdx.x * kSortThreads * kSortItems;
  for (int i = threadIdx.x; i < kSortThreads * kSortItems; i += blockDim.x) {
    const int idx = base + i;
    if (idx < n) {
      const int e = ids[idx];
      if (e >= 0 && e < num_experts) {
        atomicAdd(&s_hist[e], 1);
      } else {
        // An id outside [0, num_experts) has no expert: it is left out of the sort and recorded, so that the pass is
        // reported as invalid (every later kernel of the pass then returns at once).
        report_status(status, kStatusBadIndex, kKernelPlan, 1, 0, idx, static_cast<uint32_t>(num_experts),
                      static_cast<uint32_t>(e));
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) block_hist[e * gridDim.x + blockIdx.x] = s_hist[e];
}

__global__ void __launch_bounds__(256) sort_scan_kernel(int* block_hist, int num_experts, int num_blocks, int* counts) {
  // One thread per expert sums its blocks; then a serial scan over experts (E <= a few hundred).
  __shared__ int s_total[1024];
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    int sum = 0;
    for (int b = 0; b < num_blocks; ++b) sum += block_hist[e * num_blocks + b];
    s_total[e] = sum;
    counts[e] = sum;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < num_experts; ++e) { const int c = s_total[e]; s_total[e] = run; run += c; }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    int run = s_total[e];
    for (int b = 0; b < num_blocks; ++b) {
      const int c = block_hist[e * num_blocks + b];
      block_hist[e * num_blocks + b] = run;  // first output position of (expert e, block b)
      run += c;
    }
  }
}

__global__ void __launch_bounds__(kSortThreads) sort_scatter_kernel(const int* ids, int n, int num_experts,
                                                                  const int* block_off, int* order, int* inv_order) {
  // Stable inside the block: a thread owns kSortItems CONSECUTIVE ids; ranks come from a per-expert
  // scan over threads (done expert by expert with ballots over the ids each thread holds).
  extern __shared__ int s_mem[];
  int* s_next = s_mem;                       // [num_experts] next output slot per expert
  int* s_ids = s_mem + num_experts;          // [kSortThreads * kSortItems]
  const int base = blockIdx.x * kSortThreads * kSortItems;
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) s_next[e] = block_off[e * gridDim.x + blockIdx.x];
  for (int i = threadIdx.x; i < kSortThreads * kSortItems; i += blockDim.x)
    s_ids[i] = (base + i < n) ? ids[base + i] : -1;
  __syncthreads();
  // Thread e walks the block's ids in order for expert e (and e + blockDim, ...): stable by construction.
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    int slot = s_next[e];
    for (int i = 0; i < kSortThreads * kSortItems; ++i) {
      if (s_ids[i] == e) {
        order[slot] = base + i;
        inv_order[base + i] = slot;
        ++slot;
      }
    }
  }
}

}  // namespace

void launch_plan_build(const PlanKernelParams& p, cudaStream_t stream) {
  plan_build_kernel<<<1, 256, 0, stream>>>(p);
}

void plan_build_host(const int* counts, int* plan, const PlanLayout& lay, int me) {
  plan_phase_a(counts, plan, lay, me, 0, 1);
  plan_phase_b(plan, lay, 0, 1);
}

size_t expert_sort_scratch_ints(int n, int num_experts) {
  const int blocks = (n + kSortThreads * kSortItems - 1) / (kSortThreads * kSortItems);
  return static_cast<size_t>(blocks > 0 ? blocks : 1) * num_experts;
}

void launch_expert_sort(const int* expert_ids, int n, int num_experts, int* order, int* inv_order, int* counts,
                        int* scratch, cudaStream_t stream, StatusBlock* status) {
  int blocks = (n + kSortThreads * kSortItems - 1) / (kSortThreads * kSortItems);
  if (blocks < 1) blocks = 1;
  sort_hist_kernel<<<blocks, kSortThreads, num_experts * sizeof(int), stream>>>(expert_ids, n, num_experts, scratch,
                                                                                status);
  sort_scan_kernel<<<1, 256, 0, stream>>>(scratch, num_experts, blocks, counts);
  sort_scatter_kernel<<<blocks, kSortThreads, (num_experts + kSortThreads * kSortItems) * sizeof(int), stream>>>(
      expert_ids, n, num_experts, scratch, order, inv_order);
}

}  // namespace cem
