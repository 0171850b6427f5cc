// Plan kernel (single CTA) and expert sort.
#include "plan_kernel.cuh"

#include "../common/umma.cuh"

namespace cem {

namespace {

// Exclusive prefix sum of `v` over the warp's lanes; `total` receives the warp's sum.
__device__ __forceinline__ int warp_exclusive_scan(int v, int lane, int* total) {
  int inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += up;
  }
  *total = __shfl_sync(0xffffffffu, inc, 31);
  return inc - v;
}

// Per-pass sums on the device (what `plan_phase_a` computes with one loop nest per value): every sum the tables need is
// a prefix of a row of the traffic matrix or of the per-receiver expert totals, so the block first builds those prefix
// tables in shared memory (one thread per row, 2 P + 1 rows of at most P * L values), then every value is a lookup plus
// at most P additions. `rowsum[r][l]`: rows expert l of rank r receives; `ebegin[r][l]`: where they start in r's stream;
// `prefix[s][q]`: copies of source s that sort before its q-th (receiver, expert) pair.
__device__ void plan_phase_a_block(const int* counts, int* plan, const PlanLayout& y, int me, int* rowsum, int* ebegin,
                                   int* prefix) {
  const int P = y.P, L = y.L, n = P * L;
  const int tid = threadIdx.x, nthreads = blockDim.x;
  for (int i = tid; i < n; i += nthreads) {
    int sum = 0;
    for (int s = 0; s < P; ++s) sum += counts[s * n + i];
    rowsum[i] = sum;
  }
  __syncthreads();
  for (int row = tid; row < 2 * P; row += nthreads) {
    if (row < P) {  // exclusive scan of one receiver's expert totals
      int run = 0;
      for (int l = 0; l < L; ++l) { ebegin[row * L + l] = run; run += rowsum[row * L + l]; }
    } else {        // exclusive scan of one source's row of the traffic matrix
      const int s = row - P;
      int run = 0;
      for (int q = 0; q < n; ++q) { prefix[s * n + q] = run; run += counts[s * n + q]; }
    }
  }
  __syncthreads();
  for (int i = tid; i < n; i += nthreads) {
    const int a = i / L, l = i - a * L;  // a is the receiver r (sender view) or the source s (receiver view)
    int seg_start = ebegin[a * L + l];
    for (int s = 0; s < me; ++s) seg_start += counts[s * n + a * L + l];
    int in_start = ebegin[me * L + l];
    for (int s = 0; s < a; ++s) in_start += counts[s * n + me * L + l];
    plan[y.off_send_start + i] = prefix[me * n + i];
    plan[y.off_seg_start + i] = seg_start;
    plan[y.off_seg_size + i] = counts[me * n + i];
    plan[y.off_in_start + i] = in_start;
    plan[y.off_in_size + i] = counts[a * n + me * L + l];
    plan[y.off_src_send_start + i] = prefix[a * n + me * L + l];
  }
  for (int l = tid; l < L; l += nthreads) {
    plan[y.off_expert_start + l] = ebegin[me * L + l];
    plan[y.off_expert_rows + l] = rowsum[me * L + l];
  }
  if (tid == 0) {
    int max_rows = 0, my_rows = 0;
    for (int r = 0; r < P; ++r) {
      const int rows = ebegin[r * L + L - 1] + rowsum[r * L + L - 1];
      if (rows > max_rows) max_rows = rows;
      if (r == me) my_rows = rows;
    }
    const int my_copies = prefix[me * n + n - 1] + counts[me * n + n - 1];
    const int local_end = (me + 1) * L < n ? prefix[me * n + (me + 1) * L] : my_copies;
    const int num_slices = (max_rows + y.S - 1) / y.S;
    plan[0] = num_slices;
    plan[1] = my_rows;
    plan[2] = max_rows;
    plan[3] = my_copies - (local_end - prefix[me * n + me * L]);  // copies that leave this rank
    plan[4] = num_slices > y.max_slices ? 1 : 0;
    plan[5] = my_copies;
    for (int q = 6; q < kPlanHeaderInts; ++q) plan[q] = 0;
  }
}

// Per-slice tables, one warp per slice (what `plan_phase_b` does with one thread per slice): lanes take the experts
// (then the segments) 32 at a time and a warp scan numbers their tiles (their put chunks) in expert order.
__device__ void plan_phase_b_warps(int* plan, const PlanLayout& y, const int* seg_start, const int* seg_size,
                                   const int* send_start, const int* expert_start, const int* expert_rows) {
  const int P = y.P, L = y.L, S = y.S, n = P * L;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  int num_slices = plan[0];
  if (num_slices > y.max_slices) num_slices = y.max_slices;
  for (int j = warp; j < y.max_slices; j += nwarps) {
    int num_m = 0, num_g = 0, num_p = 0, chunks = 0;
    if (j < num_slices) {
      const int lo = j * S, hi = lo + S;
      int* mt = plan + y.off_mtiles + 4 * y.max_mtiles * j;
      int* gt = plan + y.off_gtiles + 4 * y.max_gtiles * j;
      int* pt = plan + y.off_ptiles + 4 * y.max_ptiles * j;
      for (int l0 = 0; l0 < L; l0 += 32) {
        const int l = l0 + lane;
        int es = 0, er = -1, first = 0, rows = 0;
        if (l < L) {
          es = expert_start[l];
          er = expert_rows[l];
          first = plan_clip(lo, es, es + er);
          rows = plan_clip(hi, es, es + er) - first;
        }
        const int cm = (rows + kTileM - 1) / kTileM, cp = (rows + 2 * kTileM - 1) / (2 * kTileM);
        const int cg = (rows > 0 || (j == 0 && er == 0)) ? 1 : 0;
        int tm, tp, tg;
        const int em = num_m + warp_exclusive_scan(cm, lane, &tm);
        const int ep = num_p + warp_exclusive_scan(cp, lane, &tp);
        const int eg = num_g + warp_exclusive_scan(cg, lane, &tg);
        for (int t = 0; t < cm; ++t) {
          const int off = t * kTileM;
          reinterpret_cast<int4*>(mt)[em + t] =
              make_int4(l, first - lo + off, rows - off < kTileM ? rows - off : kTileM, 0);
        }
        for (int t = 0; t < cp; ++t) {
          const int off = t * 2 * kTileM;
          reinterpret_cast<int4*>(pt)[ep + t] =
              make_int4(l, first - lo + off, rows - off < 2 * kTileM ? rows - off : 2 * kTileM, 0);
        }
        if (cg) {
          reinterpret_cast<int4*>(gt)[eg] =
              rows > 0 ? make_int4(l, first - lo, rows, (es >= lo ? kGroupFirst : 0) | (es + er <= hi ? kGroupFinal : 0))
                       : make_int4(l, 0, 0, kGroupFirst | kGroupFinal);
        }
        num_m += tm;
        num_p += tp;
        num_g += tg;
      }
      int* put = plan + y.off_put + 4 * n * j;
      for (int i0 = 0; i0 < n; i0 += 32) {
        const int i = i0 + lane;
        int ss = 0, first = 0, size = 0;
        if (i < n) {
          ss = seg_start[i];
          const int sz = seg_size[i];
          first = plan_clip(lo, ss, ss + sz);
          size = plan_clip(hi, ss, ss + sz) - first;
        }
        int tc;
        const int ec = chunks + warp_exclusive_scan((size + kPutChunkRows - 1) / kPutChunkRows, lane, &tc);
        if (i < n) reinterpret_cast<int4*>(put)[i] = make_int4(send_start[i] + (first - ss), size, first - lo, ec);
        chunks += tc;
      }
    }
    if (lane == 0) {
      plan[y.off_num_mtiles + j] = num_m;
      plan[y.off_num_gtiles + j] = num_g;
      plan[y.off_num_chunks + j] = chunks;
      plan[y.off_num_ptiles + j] = num_p;
    }
  }
}

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
  // 3. tables. When the traffic matrix and the per-segment sums fit into shared memory (always, at real sizes) the block
  // works from there and the per-slice tables are built a warp per slice; the arithmetic is `plan_phase_a/b`'s.
  extern __shared__ int s_plan[];
  if (p.use_smem) {
    const int L = p.lay.L;
    int* s_counts = s_plan;
    for (int i = threadIdx.x; i < P * n; i += blockDim.x) s_counts[i] = p.counts[i];
    __syncthreads();
    // scratch of the per-pass sums: rowsum [n], ebegin [n], prefix [P * n]; the same space holds phase B's inputs after
    plan_phase_a_block(s_counts, p.plan, p.lay, p.me, s_counts + P * n, s_counts + P * n + n, s_counts + P * n + 2 * n);
    __syncthreads();
    int* s_seg_start = s_counts + P * n;
    int* s_seg_size = s_seg_start + n;
    int* s_send_start = s_seg_size + n;
    int* s_expert_start = s_send_start + n;
    int* s_expert_rows = s_expert_start + L;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      s_seg_start[i] = p.plan[p.lay.off_seg_start + i];
      s_seg_size[i] = p.plan[p.lay.off_seg_size + i];
      s_send_start[i] = p.plan[p.lay.off_send_start + i];
    }
    for (int l = threadIdx.x; l < L; l += blockDim.x) {
      s_expert_start[l] = p.plan[p.lay.off_expert_start + l];
      s_expert_rows[l] = p.plan[p.lay.off_expert_rows + l];
    }
    __syncthreads();
    plan_phase_b_warps(p.plan, p.lay, s_seg_start, s_seg_size, s_send_start, s_expert_start, s_expert_rows);
    return;
  }
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

// Stable scatter of one block's 2048 ids. A warp owns 256 CONSECUTIVE ids. (1) every warp counts its ids per expert in
// shared memory; (2) an exclusive sum over the warps, on top of the block's first slot of each expert, turns the counts
// into the first output slot of every (warp, expert); (3) each warp walks its ids 32 at a time, in order: lanes holding
// the same expert find each other with `match.any`, a lane's rank among them is the number of lower lanes, and the
// lowest lane advances the (warp, expert) slot. (The serial form below took 45 us per launch on the critical path at
// the start of every pass; this one a few.)
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortRankedMaxExperts = 1024;  // kSortWarps * experts ints of shared memory: 32 KB

__global__ void __launch_bounds__(kSortThreads) sort_scatter_kernel(const int* ids, int n, int num_experts,
                                                                  const int* block_off, int* order, int* inv_order) {
  extern __shared__ int s_slot[];  // [kSortWarps][num_experts]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int base = blockIdx.x * kSortThreads * kSortItems + warp * (kSortItems * 32);
  for (int i = threadIdx.x; i < kSortWarps * num_experts; i += blockDim.x) s_slot[i] = 0;
  __syncthreads();
  int* mine = s_slot + warp * num_experts;
  int e_of[kSortItems];
#pragma unroll
  for (int g = 0; g < kSortItems; ++g) {
    const int idx = base + g * 32 + lane;
    int e = (idx < n) ? ids[idx] : -1;
    if (e < 0 || e >= num_experts) e = -1;  // takes no part in the sort
    e_of[g] = e;
    if (e >= 0) atomicAdd(mine + e, 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    int run = block_off[e * gridDim.x + blockIdx.x];
#pragma unroll
    for (int w = 0; w < kSortWarps; ++w) {
      const int c = s_slot[w * num_experts + e];
      s_slot[w * num_experts + e] = run;
      run += c;
    }
  }
  __syncthreads();
#pragma unroll
  for (int g = 0; g < kSortItems; ++g) {
    const int e = e_of[g];
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int leader = __ffs(peers) - 1;
    int first = 0;
    if (e >= 0 && lane == leader) {
      first = mine[e];
      mine[e] = first + __popc(peers);
    }
    first = __shfl_sync(0xffffffffu, first, leader);
    if (e >= 0) {
      const int slot = first + __popc(peers & ((1u << lane) - 1u));
      const int idx = base + g * 32 + lane;
      order[slot] = idx;
      inv_order[idx] = slot;
    }
    __syncwarp();  // the next group's leaders see this group's slot updates
  }
}

__global__ void __launch_bounds__(kSortThreads) sort_scatter_serial_kernel(const int* ids, int n, int num_experts,
                                                                  const int* block_off, int* order, int* inv_order) {
  // Fallback for more experts than the ranked kernel below has shared memory for: one thread per expert walks the
  // block's ids in order.
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

void launch_plan_build(const PlanKernelParams& p_in, cudaStream_t stream) {
  PlanKernelParams p = p_in;
  const int n = p.lay.P * p.lay.L;
  // the matrix [P * n], then the larger of phase A's scratch (2 n + P * n) and phase B's inputs (3 n + 2 L)
  const size_t after = static_cast<size_t>(p.lay.P) * n + 2 * static_cast<size_t>(n) + 2 * p.lay.L + n;
  const size_t smem = sizeof(int) * (static_cast<size_t>(p.lay.P) * n + after);
  p.use_smem = smem <= 40 * 1024 ? 1 : 0;  // 256 experts on 8 ranks need 20 KB; anything larger takes the serial path
  plan_build_kernel<<<1, 256, p.use_smem ? smem : 0, stream>>>(p);
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
  if (num_experts <= kSortRankedMaxExperts)
    sort_scatter_kernel<<<blocks, kSortThreads, kSortWarps * num_experts * sizeof(int), stream>>>(
        expert_ids, n, num_experts, scratch, order, inv_order);
  else
    sort_scatter_serial_kernel<<<blocks, kSortThreads, (num_experts + kSortThreads * kSortItems) * sizeof(int),
                                 stream>>>(expert_ids, n, num_experts, scratch, order, inv_order);
}

}  // namespace cem
