// Dispatch put, credits, combine reduce.
//
// dispatch_put replaces three things of the reference at once: the send-order gather
// (src/chunked_moe/moe.py:91-93), the wire quantisation (moe.py:56-63) and the slice exchange
// (transport/nvshmem.py:125-177 / ragged_all_to_all). A warp takes a chunk of up to
// kPutChunkRows rows of one (receiver, expert) segment, reads each row straight from x[token]
// (no [T*K, D] send buffer is ever materialised), stores it with 16-byte vector stores into the
// expert-major position of the receiver's S-row slice buffer over NVLink, and then releases
// the row count to the receiver's per-(source, expert) arrival counter. Receivers never take
// part in the transfer; their GEMM producer warps acquire the counters.
//
// Protocol invariants:
//   * arrival counters only grow (cumulative rows per (source, expert)); a pass's targets are
//     base + rows expected so far, so nothing is ever reset and stale values are detectable;
//   * slice buffers are double buffered by the global slice sequence number; before writing
//     sequence q a sender waits until the receiver's credit says q-2 has been consumed;
//   * every wait is bounded and reports through the status block.
#include "comm_kernels.cuh"

#include <cuda_fp8.h>

#include "../common/umma.cuh"

namespace cem {

namespace {

constexpr int kPutThreads = 512;

__device__ __forceinline__ int find_segment(const int4* put, int n, int chunk) {
  // Last segment whose chunk prefix is <= chunk (empty segments share a prefix with their successor).
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (put[mid].w <= chunk) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ void copy_row_bf16(const __nv_bfloat16* src, __nv_bfloat16* dst, int hidden, int lane) {
  const int units = hidden >> 3;  // 16-byte units
  const int4* s = reinterpret_cast<const int4*>(src);
  int4* d = reinterpret_cast<int4*>(dst);
  int u = lane;
  for (; u + 96 < units; u += 128) {
    const int4 a = ld_nc_v4(s + u), b = ld_nc_v4(s + u + 32), c = ld_nc_v4(s + u + 64), e = ld_nc_v4(s + u + 96);
    d[u] = a; d[u + 32] = b; d[u + 64] = c; d[u + 96] = e;
  }
  for (; u < units; u += 32) d[u] = ld_nc_v4(s + u);
}

// Quantises one row to e4m3 with a scale per 128 columns. 16 lanes cover one block (8 values each).
__device__ __forceinline__ void put_row_fp8(const __nv_bfloat16* src, uint8_t* dq, float* ds, int hidden, int lane) {
  const int units = hidden >> 3;
  const int4* s = reinterpret_cast<const int4*>(src);
  for (int u0 = 0; u0 < units; u0 += 32) {
    const int u = u0 + lane;
    float v[8];
    if (u < units) {
      const int4 raw = ld_nc_v4(s + u);
      const uint32_t wds[4] = {static_cast<uint32_t>(raw.x), static_cast<uint32_t>(raw.y),
                               static_cast<uint32_t>(raw.z), static_cast<uint32_t>(raw.w)};
#pragma unroll
      for (int i = 0; i < 4; ++i) { v[2 * i] = bf16_lo(wds[i]); v[2 * i + 1] = bf16_hi(wds[i]); }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = fmaxf(amax, 1e-12f) * (1.0f / 448.0f);
    const float inv = 1.0f / scale;
    if (u < units) {
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t b0 = __nv_cvt_float_to_fp8(v[i] * inv, __NV_SATFINITE, __NV_E4M3);
        const uint32_t b1 = __nv_cvt_float_to_fp8(v[4 + i] * inv, __NV_SATFINITE, __NV_E4M3);
        lo |= b0 << (8 * i);
        hi |= b1 << (8 * i);
      }
      *reinterpret_cast<uint2*>(dq + static_cast<size_t>(u) * 8) = make_uint2(lo, hi);
      if ((lane & 15) == 0) ds[u >> 4] = scale;
    }
  }
}

__global__ void __launch_bounds__(kPutThreads) dispatch_put_kernel(const PutParams p) {
  __shared__ int s_abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_seg = p.lay.P * p.lay.L;
  if (threadIdx.x == 0) s_abort = (p.status != nullptr && p.status->code != 0) ? 1 : 0;
  __syncthreads();
  if (s_abort) return;  // an earlier kernel of this pass already gave up
  // Buffer reuse: sequence q overwrites what sequence q-2 used on every receiver.
  if (p.seq >= 2 && threadIdx.x < p.lay.P) {
    uint32_t seen = 0;
    if (!spin_until_reached(p.credit + threadIdx.x, p.seq - 1, p.spin_limit, &seen)) {
      report_status(p.status, kStatusCreditTimeout, kKernelPut, 0, static_cast<int>(p.seq), threadIdx.x, p.seq - 1, seen);
      s_abort = 1;
    }
  }
  __syncthreads();
  if (s_abort) return;

  const int num_chunks = p.plan[p.lay.off_num_chunks + p.slice];
  const int4* put = reinterpret_cast<const int4*>(p.plan + p.lay.off_put + 4 * n_seg * p.slice);
  const int buf = static_cast<int>(p.seq & 1u);
  const int S = p.lay.S, D = p.hidden;
  const int warps_total = gridDim.x * (kPutThreads / 32);
  // Arrival releases are batched: a system-scope fence drains this warp's stores over NVLink, so one fence covers
  // up to kPendingSignals chunks instead of one (lane i of the warp keeps pending signal i).
  constexpr int kPendingSignals = 8;
  uint32_t* pend_ptr = nullptr;
  uint32_t pend_cnt = 0;
  int pending = 0;
  auto flush = [&]() {
    __syncwarp();
    if (lane < pending) {
      __threadfence_system();
      red_add_release_sys(pend_ptr, pend_cnt);
    }
    pending = 0;
  };
  for (int c = blockIdx.x * (kPutThreads / 32) + warp; c < num_chunks; c += warps_total) {
    const int seg = find_segment(put, n_seg, c);
    const int4 e = put[seg];  // {send-order offset, rows, dest row, chunk prefix}
    const int r = seg / p.lay.L, l = seg - r * p.lay.L;
    const int first = (c - e.w) * kPutChunkRows;
    const int rows = min(kPutChunkRows, e.y - first);
    for (int rr = 0; rr < rows; ++rr) {
      const int flat = p.order[e.x + first + rr];
      const int token = flat / p.top_k;
      // Index check (warp-uniform): a send-order entry outside the token range or a destination row outside the
      // slice buffer is recorded and the row is skipped, never dereferenced. The arrival is still signalled, so
      // nothing waits for the row; the recorded status tells the host that the pass is invalid.
      if (flat < 0 || token >= p.num_tokens || e.z + first + rr >= S) {
        if (lane == 0)
          report_status(p.status, kStatusBadIndex, kKernelPut, 0, p.slice, e.x + first + rr,
                        static_cast<uint32_t>(p.num_tokens), static_cast<uint32_t>(token));
        continue;
      }
      const size_t drow = static_cast<size_t>(buf) * S + e.z + first + rr;
      if (p.peer_xq == nullptr) {
        copy_row_bf16(p.x + static_cast<size_t>(token) * D, p.peer_x[r] + drow * D, D, lane);
        if (p.g != nullptr) copy_row_bf16(p.g + static_cast<size_t>(token) * D, p.peer_g[r] + drow * D, D, lane);
      } else {
        put_row_fp8(p.x + static_cast<size_t>(token) * D, p.peer_xq[r] + drow * D, p.peer_xs[r] + drow * (D >> 7), D, lane);
        if (p.g != nullptr)
          put_row_fp8(p.g + static_cast<size_t>(token) * D, p.peer_gq[r] + drow * D, p.peer_gs[r] + drow * (D >> 7), D, lane);
      }
      if (lane == 0) p.peer_w[r][drow] = p.w_flat[flat];
    }
    if (lane == pending) {
      pend_ptr = p.peer_arrive[r] + p.me * p.lay.L + l;
      pend_cnt = static_cast<uint32_t>(rows);
    }
    if (++pending == kPendingSignals) flush();
  }
  flush();
}

__global__ void slice_done_kernel(uint32_t* const* peer_credit, int num_ranks, int me, uint32_t seq) {
  if (threadIdx.x < num_ranks) st_release_sys(peer_credit[threadIdx.x] + me, seq + 1);
}

__global__ void pass_begin_kernel(const int* plan, PlanLayout lay, uint32_t* expected_total, uint32_t* pass_base,
                                  uint32_t* ready_total, uint32_t* ready_base) {
  const int n = lay.P * lay.L;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const uint32_t base = expected_total[i];
    pass_base[i] = base;
    expected_total[i] = base + static_cast<uint32_t>(plan[lay.off_in_size + i]);
  }
  if (ready_total != nullptr) {
    for (int l = threadIdx.x; l < lay.L; l += blockDim.x) {
      const uint32_t base = ready_total[l];
      ready_base[l] = base;
      ready_total[l] = base + static_cast<uint32_t>(plan[lay.off_expert_rows + l]);
    }
  }
}

__global__ void __launch_bounds__(256) combine_reduce_kernel(const CombineParams p) {
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    s_abort = (p.status != nullptr && p.status->code != 0) ? 1 : 0;
    uint32_t seen = 0;
    if (!s_abort && !spin_until_reached(p.count, p.target, p.spin_limit, &seen)) {
      report_status(p.status, kStatusReturnTimeout, kKernelCombineReduce, 0, 0, 0, p.target, seen);
      s_abort = 1;
    }
  }
  __syncthreads();
  if (s_abort) return;
  const int units = p.hidden >> 3;
  for (int t = blockIdx.x; t < p.num_tokens; t += gridDim.x) {
    for (int u = threadIdx.x; u < units; u += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
      for (int k = 0; k < p.top_k; ++k) {  // fixed k order: bitwise reproducible
        const int pos = p.inv_order[t * p.top_k + k];
        const size_t at = p.blocked ? (static_cast<size_t>(u >> 5) * p.ret_rows + pos) * 256 + (((u & 31) ^ (pos & 7)) << 3)
                                    : static_cast<size_t>(pos) * p.hidden + u * 8;
        const int4 raw = *reinterpret_cast<const int4*>(p.rows + at);
        const uint32_t wds[4] = {static_cast<uint32_t>(raw.x), static_cast<uint32_t>(raw.y),
                                 static_cast<uint32_t>(raw.z), static_cast<uint32_t>(raw.w)};
#pragma unroll
        for (int i = 0; i < 4; ++i) { acc[2 * i] += bf16_lo(wds[i]); acc[2 * i + 1] += bf16_hi(wds[i]); }
      }
      *reinterpret_cast<int4*>(p.out + static_cast<size_t>(t) * p.hidden + u * 8) =
          make_int4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]),
                    pack_bf16(acc[6], acc[7]));
    }
    if (p.d_weights != nullptr && threadIdx.x < p.top_k) {
      const int flat = t * p.top_k + threadIdx.x;
      p.d_weights[flat] = p.dw_rows[p.inv_order[flat]];
    }
  }
}

// Expands one e4m3 row with its 1x128 block scales into bf16; the CTA's threads stride over 8-value units.
__device__ __forceinline__ void dequant_row(const uint8_t* q, const float* scales, __nv_bfloat16* out, int row,
                                            int hidden) {
  const int units = hidden >> 3;
  const uint8_t* qrow = q + static_cast<size_t>(row) * hidden;
  const float* srow = scales + static_cast<size_t>(row) * (hidden >> 7);
  __nv_bfloat16* orow = out + static_cast<size_t>(row) * hidden;
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
    const uint2 raw = *reinterpret_cast<const uint2*>(qrow + static_cast<size_t>(u) * 8);
    const float scale = srow[u >> 4];
    float v[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half_raw h0 = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>((raw.x >> (8 * i)) & 0xFF), __NV_E4M3);
      const __half_raw h1 = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>((raw.y >> (8 * i)) & 0xFF), __NV_E4M3);
      v[i] = __half2float(*reinterpret_cast<const __half*>(&h0)) * scale;
      v[4 + i] = __half2float(*reinterpret_cast<const __half*>(&h1)) * scale;
    }
    *reinterpret_cast<int4*>(orow + static_cast<size_t>(u) * 8) =
        make_int4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
  }
}

__global__ void __launch_bounds__(256) dequant_slice_kernel(const DequantParams p) {
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = (p.status != nullptr && p.status->code != 0) ? 1 : 0;
  __syncthreads();
  if (s_abort) return;
  const int lo = p.slice * p.lay.S, hi = lo + p.lay.S;
  for (int l = 0; l < p.lay.L; ++l) {
    const int es = p.plan[p.lay.off_expert_start + l], er = p.plan[p.lay.off_expert_rows + l];
    const int first = plan_clip(lo, es, es + er), last = plan_clip(hi, es, es + er);
    if (last <= first) continue;
    // This expert's rows of the slice have arrived from every source (thread s watches source s).
    if (threadIdx.x < p.lay.P) {
      const int i = threadIdx.x * p.lay.L + l;
      const int through = plan_clip(hi - p.plan[p.lay.off_in_start + i], 0, p.plan[p.lay.off_in_size + i]);
      const uint32_t target = p.pass_base[i] + static_cast<uint32_t>(through);
      uint32_t seen = 0;
      if (!spin_until_reached(p.arrive + i, target, p.spin_limit, &seen)) {
        report_status(p.status, kStatusArrivalTimeout, kKernelPut, 1, p.slice, i, target, seen);
        s_abort = 1;
      }
    }
    __syncthreads();
    if (s_abort) return;
    // Slice rows [first - lo, last - lo); this CTA takes every gridDim.x-th of them.
    uint32_t mine = 0;
    for (int r = first - lo + blockIdx.x; r < last - lo; r += gridDim.x, ++mine) {
      dequant_row(p.xq, p.xs, p.x, r, p.hidden);
      if (p.gq != nullptr) dequant_row(p.gq, p.gs, p.g, r, p.hidden);
    }
    __syncthreads();  // all of this CTA's stores for the expert are issued before one thread releases them
    if (threadIdx.x == 0 && mine > 0) {
      __threadfence();
      atomicAdd(p.ready + l, mine);
    }
  }
}

__global__ void wait_probe_kernel(const uint32_t* flag, uint32_t target, uint32_t spin_limit, StatusBlock* status) {
  uint32_t seen = 0;
  if (!spin_until_reached(flag, target, spin_limit, &seen))
    report_status(status, kStatusArrivalTimeout, kKernelWaitProbe, 0, 0, 0, target, seen);
}

}  // namespace

void launch_dispatch_put(const PutParams& p, int grid, cudaStream_t stream) {
  dispatch_put_kernel<<<grid, kPutThreads, 0, stream>>>(p);
}

void launch_slice_done(uint32_t* const* peer_credit, int num_ranks, int me, uint32_t seq, cudaStream_t stream) {
  slice_done_kernel<<<1, 32, 0, stream>>>(peer_credit, num_ranks, me, seq);
}

void launch_pass_begin(const int* plan, PlanLayout lay, uint32_t* expected_total, uint32_t* pass_base,
                       uint32_t* ready_total, uint32_t* ready_base, cudaStream_t stream) {
  pass_begin_kernel<<<1, 256, 0, stream>>>(plan, lay, expected_total, pass_base, ready_total, ready_base);
}

void launch_combine_reduce(const CombineParams& p, cudaStream_t stream) {
  int grid = p.num_tokens < 1184 ? p.num_tokens : 1184;  // 8 CTAs per SM on 148 SMs
  if (grid < 1) grid = 1;
  combine_reduce_kernel<<<grid, 256, 0, stream>>>(p);
}

void launch_dequant_slice(const DequantParams& p, cudaStream_t stream) {
  // Every CTA visits every expert of the slice and waits for its arrival, so ALL CTAs must be resident at once for
  // an expert's rows to be released while later experts are still arriving: 72 CTAs of 256 threads fit on the dozen
  // SMs the up-projection GEMM leaves free on the fp8 wire (8 such CTAs per SM).
  dequant_slice_kernel<<<72, 256, 0, stream>>>(p);
}

void launch_wait_probe(const uint32_t* flag, uint32_t target, uint32_t spin_limit, StatusBlock* status,
                       cudaStream_t stream) {
  wait_probe_kernel<<<1, 1, 0, stream>>>(flag, target, spin_limit, status);
}

}  // namespace cem
