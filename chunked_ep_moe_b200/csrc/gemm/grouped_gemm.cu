// Grouped GEMM engine for sm_100a: persistent, warp-specialised, tcgen05 MMA with TMEM accumulators.
//
//   warp 0      TMA producer. Walks this CTA's tiles, (for the dispatch consumer) acquires the
//               arrival counters of the tile's expert, then streams A/B k-blocks into a 4-stage
//               shared-memory ring with cp.async.bulk.tensor (this CTA's shared memory only).
//   warp 1      MMA issuer. One lane issues tcgen05.mma (128x256x16, bf16 -> fp32 in TMEM) and
//               commits to the ring's empty barriers and to the accumulator-full barrier.
//   warps 2-5   Epilogue. Each warp owns 32 TMEM lanes (= 32 tile rows, one row per thread),
//               reads the accumulator with tcgen05.ld and applies the mode's fused epilogue.
//
// The accumulator is double buffered (2 x 256 TMEM columns) so the epilogue of tile i overlaps
// the MMAs of tile i+1. Ragged row groups come from the plan's compact tile list; rows of a tile
// past its group are computed but never stored, and weight-gradient k-blocks that straddle a
// group end are zero-filled in shared memory (select, not multiply, so NaN padding cannot leak).
//
// What each mode replaces in the reference is listed next to `GemmMode` in grouped_gemm.cuh
// (reference kernels: src/chunked_moe/kernels/fused_expert.py:102-352).
#include "grouped_gemm.cuh"

#include "../common/umma.cuh"

namespace cem {

namespace {

template <int MODE>
struct ModeTraits {
  static constexpr bool kAMn = (MODE == kModeTgmm);  // A is MN-major (contraction over rows)
  static constexpr bool kBMn = (MODE == kModeSwiglu || MODE == kModeDownFwd || MODE == kModeDownDw || MODE == kModeTgmm);
  static constexpr bool kCombine = (MODE == kModeDownFwd || MODE == kModeDx);
};

struct Tile {
  int g;      // local expert
  int row0;   // first slice row of the tile (gmm) / of the group (tgmm)
  int nrows;  // valid rows of the tile / rows of the group
  int flags;  // tgmm: kGroupFirst | kGroupFinal
  int m;      // tgmm: row tile of the weight gradient
  int n;      // column tile
  int kblocks;
};

template <int MODE>
__device__ __forceinline__ Tile decode_tile(const GemmParams& p, int t, int num_entries) {
  Tile tl;
  if constexpr (MODE == kModeTgmm) {
    const int per_group = p.m_tiles * p.n_tiles;
    const int gi = t / per_group, rem = t - gi * per_group;
    const int4 e = reinterpret_cast<const int4*>(p.plan + p.lay.off_gtiles + 4 * p.lay.max_gtiles * p.slice)[gi];
    tl.g = e.x; tl.row0 = e.y; tl.nrows = e.z; tl.flags = e.w;
    tl.m = rem / p.n_tiles; tl.n = rem - tl.m * p.n_tiles;
    tl.kblocks = (e.z + kBlockK - 1) / kBlockK;
  } else {
    // Banded raster: `kRasterBand` consecutive row tiles sweep all column tiles together.
    const int band_tiles = kRasterBand * p.n_tiles;
    const int band = t / band_tiles, rem = t - band * band_tiles;
    int width = num_entries - band * kRasterBand;
    width = width > kRasterBand ? kRasterBand : width;
    tl.n = rem / width;
    const int mi = band * kRasterBand + (rem - tl.n * width);
    const int4 e = reinterpret_cast<const int4*>(p.plan + p.lay.off_mtiles + 4 * p.lay.max_mtiles * p.slice)[mi];
    tl.g = e.x; tl.row0 = e.y; tl.nrows = e.z; tl.flags = 0; tl.m = mi;
    tl.kblocks = p.k_blocks;
  }
  return tl;
}

// Source rank and send-order position of slice row `grow` of expert `g` (combine target).
__device__ __forceinline__ void resolve_source(const GemmParams& p, int g, int grow, int* src, int* pos) {
  const int stream_row = p.slice * p.lay.S + grow;
  const int* in_start = p.plan + p.lay.off_in_start;
  const int* in_size = p.plan + p.lay.off_in_size;
  const int* sss = p.plan + p.lay.off_src_send_start;
  *src = -1;
  *pos = 0;
  for (int s = 0; s < p.lay.P; ++s) {
    const int i = s * p.lay.L + g;
    const int st = in_start[i];
    if (stream_row >= st && stream_row < st + in_size[i]) {
      *src = s;
      *pos = sss[i] + (stream_row - st);
    }
  }
}

// Issues the TMA loads of one k-block of a tile into a pipeline stage (completing on `bar`).
// (An L2 prefetch cursor running 8 k-blocks ahead of these loads was measured and made the GEMM
// modes ~14% slower at DeepSeek-V3 sizes, so there is none.)
template <int MODE>
__device__ __forceinline__ void issue_kblock(const GemmParams& p, const Tile& tl, int kb, const CUtensorMap* map_a,
                                             const CUtensorMap* map_b, uint32_t sa, uint32_t sb, uint32_t bar) {
  using Traits = ModeTraits<MODE>;
  auto go = [&](const CUtensorMap* map, uint32_t dst, int x, int y) { tma_load_2d(dst, map, bar, x, y); };
  if constexpr (Traits::kAMn) {
    // lhs [S, M]: k runs over rows; two 64-column chunks of the 128-wide row tile.
    go(map_a, sa, tl.m * kBlockM, tl.row0 + kb * kBlockK);
    go(map_a, sa + 8192, tl.m * kBlockM + 64, tl.row0 + kb * kBlockK);
  } else {
    go(map_a, sa, kb * kBlockK, tl.row0);
  }
  if constexpr (MODE == kModeTgmm) {
#pragma unroll
    for (int c = 0; c < 4; ++c) go(map_b, sb + c * 8192, tl.n * kBlockN + c * 64, tl.row0 + kb * kBlockK);
  } else if constexpr (Traits::kBMn) {
    // weights [L*K, N]: four 64-column chunks of the 256-wide column tile.
#pragma unroll
    for (int c = 0; c < 4; ++c)
      go(map_b, sb + c * 8192, tl.n * kBlockN + c * 64, tl.g * p.b_group_rows + kb * kBlockK);
  } else {
    // weights [L*N, K] read as K-major B: 256 rows x 64 k.
    go(map_b, sb, kb * kBlockK, tl.g * p.b_group_rows + tl.n * kBlockN);
  }
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + __expf(-g)); }

template <int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b) {
  using Traits = ModeTraits<MODE>;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzled tiles want 1024-byte aligned bases.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t staging_base = smem_base + kStages * kStageBytes;
  uint8_t* staging_gen = smem_gen + kStages * kStageBytes;
  const uint32_t bar_base = staging_base + kStagingBytes;
  // barriers: full[kStages], empty[kStages], acc_full[2], acc_empty[2], drain; then tmem slot, abort flag
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto acc_full_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };
  auto acc_empty_bar = [&](int s) { return bar_base + 8u * (2 * kStages + 2 + s); };
  const uint32_t drain_bar = bar_base + 8u * (2 * kStages + 4);
  const uint32_t tmem_slot = bar_base + 8u * (2 * kStages + 5);
  volatile uint32_t* tmem_slot_gen =
      reinterpret_cast<volatile uint32_t*>(staging_gen + kStagingBytes + 8 * (2 * kStages + 5));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(staging_gen + kStagingBytes + 8 * (2 * kStages + 5) + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(acc_full_bar(s), 1);
      mbar_init(acc_empty_bar(s), 4);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;

  const int num_entries = (MODE == kModeTgmm) ? p.plan[p.lay.off_num_gtiles + p.slice]
                                              : p.plan[p.lay.off_num_mtiles + p.slice];
  const int num_tiles = (MODE == kModeTgmm) ? num_entries * p.m_tiles * p.n_tiles : num_entries * p.n_tiles;

  if (warp == 0) {
    // ================================ TMA producer ==========================================
    uint32_t it = 0;
    int waited_expert = -1;
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
      const Tile tl = decode_tile<MODE>(p, t, num_entries);
      if constexpr (MODE == kModeSwiglu) {
        if (p.arrive != nullptr && tl.g != waited_expert) {
          // Rows of expert g come from every source rank; lane s watches source s.
          bool ok = true;
          uint32_t seen = 0, target = 0;
          if (lane < p.lay.P) {
            const int i = lane * p.lay.L + tl.g;
            const int through = plan_clip((p.slice + 1) * p.lay.S - p.plan[p.lay.off_in_start + i], 0,
                                          p.plan[p.lay.off_in_size + i]);
            target = p.pass_base[i] + static_cast<uint32_t>(through);
            ok = spin_until_reached(p.arrive + i, target, p.spin_limit, &seen);
            if (!ok) {
              report_status(p.status, kStatusArrivalTimeout, kKernelGemm, MODE, p.slice, i, target, seen);
              *abort_flag = 1;
            }
          }
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          waited_expert = tl.g;
          fence_proxy_async_all();  // arrived rows were written through the generic proxy; TMA reads them next
        }
      }
      if (lane == 0) {
        for (int kb = 0; kb < tl.kblocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, p.mbar_limit)) {
            report_status(p.status, kStatusMbarTimeout, kKernelGemm, MODE, t, 100 + s, 0, 0);
            *abort_flag = 1;
            break;
          }
          const uint32_t sa = smem_base + s * kStageBytes;
          const uint32_t sb = sa + kStageBytesA;
          mbar_expect_tx(full_bar(s), kStageBytes);
          issue_kblock<MODE>(p, tl, kb, &map_a, &map_b, sa, sb, full_bar(s));
        }
      }
      __syncwarp();
    }
    if (lane == 0 && *abort_flag) {
      // Unwinding: let our copies in flight land before the CTA gives its shared memory back.
      for (int s = 0; s < kStages; ++s) {
        if (it > static_cast<uint32_t>(s)) {
          const uint32_t last = it - 1 - ((it - 1 - s) % kStages);  // last iteration that used stage s
          mbar_wait(full_bar(s), (last / kStages) & 1u, p.mbar_limit);
        }
      }
    }
  } else if (warp == 1) {
    // ================================ MMA issuer ============================================
    constexpr uint32_t idesc = make_instr_desc_bf16(kBlockM, kBlockN, Traits::kAMn, Traits::kBMn);
    uint32_t it = 0, tcount = 0;
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x, ++tcount) {
      const Tile tl = decode_tile<MODE>(p, t, num_entries);
      const int as = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1u;
      bool ok = true;
      if (lane == 0) {
        ok = mbar_wait(acc_empty_bar(as), aph ^ 1u, p.mbar_limit);
        if (!ok) {
          report_status(p.status, kStatusMbarTimeout, kKernelGemm, MODE, t, 200 + as, 0, 0);
          *abort_flag = 1;
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tcgen05_fence_after_sync();
      const uint32_t tmem_d = tmem_base + as * kBlockN;
      for (int kb = 0; kb < tl.kblocks; ++kb, ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1u;
        if (lane == 0) {
          ok = mbar_wait(full_bar(s), ph, p.mbar_limit);
          if (!ok) {
            report_status(p.status, kStatusMbarTimeout, kKernelGemm, MODE, t, 300 + s, 0, 0);
            *abort_flag = 1;
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        const uint32_t sa = smem_base + s * kStageBytes;
        const uint32_t sb = sa + kStageBytesA;
        int ksteps = kBlockK / kUmmaK;
        if constexpr (MODE == kModeTgmm) {
          const int valid = tl.nrows - kb * kBlockK;  // rows of this k-block inside the group
          if (valid < kBlockK) {
            ksteps = (valid + kUmmaK - 1) / kUmmaK;
            // Rows [valid, ksteps*16) belong to the next group (or are padding): zero them in
            // both operands. Each k row is one 128-byte line per 64-column chunk.
            uint8_t* ga = smem_gen + s * kStageBytes;
            const int zrows = ksteps * kUmmaK - valid;
            for (int idx = lane; idx < zrows * 6 * 8; idx += 32) {
              const int v16 = idx & 7, line = idx >> 3;
              const int chunk = line % 6, r = valid + line / 6;
              *reinterpret_cast<int4*>(ga + chunk * 8192 + r * 128 + v16 * 16) = make_int4(0, 0, 0, 0);
            }
            fence_proxy_async_smem();
            __syncwarp();
          }
        }
        tcgen05_fence_after_sync();
        if (lane == 0) {
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            if (k < ksteps) {
              // K-major: 16 bf16 = 32 bytes along the swizzled row. MN-major: 16 k rows = 2048 bytes.
              const uint64_t da = Traits::kAMn ? make_smem_desc(sa + k * 2048, 8192, 1024)
                                               : make_smem_desc(sa + k * 32, 16, 1024);
              const uint64_t db = Traits::kBMn ? make_smem_desc(sb + k * 2048, 8192, 1024)
                                               : make_smem_desc(sb + k * 32, 16, 1024);
              umma_bf16(tmem_d, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
          }
          umma_commit(empty_bar(s));  // frees the stage once these MMAs have read it
        }
        __syncwarp();
      }
      if (!ok) break;
      if (lane == 0) {
        if (tl.kblocks > 0) {
          umma_commit(acc_full_bar(as));
        } else {
          mbar_arrive(acc_full_bar(as));  // empty group: nothing was issued, the epilogue writes zeros
        }
      }
      __syncwarp();
    }
    if (lane == 0 && *abort_flag) {
      // Unwinding: let the MMAs already issued finish before TMEM is freed.
      umma_commit(drain_bar);
      mbar_wait(drain_bar, 0, p.mbar_limit);
    }
  } else {
    // ================================ epilogue ==============================================
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;       // tile row owned by this thread
    uint8_t* stage_gen = staging_gen + (warp - 2) * 8192;
    uint32_t tcount = 0;
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x, ++tcount) {
      const Tile tl = decode_tile<MODE>(p, t, num_entries);
      const int as = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1u;
      bool ok = mbar_wait(acc_full_bar(as), aph, p.mbar_limit);
      if (!ok) {
        report_status(p.status, kStatusMbarTimeout, kKernelGemm, MODE, t, 400 + as, 0, 0);
        *abort_flag = 1;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after_sync();
      const uint32_t tacc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * kBlockN;
      const int grow = tl.row0 + row;
      const bool valid = (MODE == kModeTgmm) ? true : (row < tl.nrows);
      uint32_t r[32];

      if constexpr (MODE == kModeSwiglu) {
        uint32_t u[32];
        __nv_bfloat16* act_row = p.out0 + static_cast<size_t>(grow) * p.ld0 + tl.n * (kBlockN / 2);
        __nv_bfloat16* h_row = p.out1 ? p.out1 + static_cast<size_t>(grow) * p.ld1 + tl.n * kBlockN : nullptr;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          const int f_local = c * 32;
          const int b = f_local / p.stripe, off = f_local - b * p.stripe;
          const int gcol = 2 * b * p.stripe + off, ucol = gcol + p.stripe;
          tmem_ld_32x32(tacc + gcol, r);
          tmem_ld_32x32(tacc + ucol, u);
          tmem_ld_wait();
          if (valid) {
            uint32_t o[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float g0 = __uint_as_float(r[2 * i]), g1 = __uint_as_float(r[2 * i + 1]);
              const float u0 = __uint_as_float(u[2 * i]), u1 = __uint_as_float(u[2 * i + 1]);
              o[i] = pack_bf16(silu_f(g0) * u0, silu_f(g1) * u1);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<int4*>(act_row + f_local + 8 * i) = make_int4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
            if (h_row != nullptr) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                *reinterpret_cast<int4*>(h_row + gcol + 8 * i) =
                    make_int4(pack_bf16(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1])),
                              pack_bf16(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3])),
                              pack_bf16(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5])),
                              pack_bf16(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7])));
                *reinterpret_cast<int4*>(h_row + ucol + 8 * i) =
                    make_int4(pack_bf16(__uint_as_float(u[8 * i]), __uint_as_float(u[8 * i + 1])),
                              pack_bf16(__uint_as_float(u[8 * i + 2]), __uint_as_float(u[8 * i + 3])),
                              pack_bf16(__uint_as_float(u[8 * i + 4]), __uint_as_float(u[8 * i + 5])),
                              pack_bf16(__uint_as_float(u[8 * i + 6]), __uint_as_float(u[8 * i + 7])));
              }
            }
          }
        }
      } else if constexpr (Traits::kCombine) {
        // Rows go back to the rank they came from, at their send-order position.
        int src = -1, pos = 0;
        if (valid) resolve_source(p, tl.g, grow, &src, &pos);
        float w = 1.0f;
        if constexpr (MODE == kModeDownFwd) w = valid ? p.row_w[grow] : 0.0f;
        unsigned long long dst = 0;
        if (src >= 0)
          dst = reinterpret_cast<unsigned long long>(p.peer_rows[src] + static_cast<size_t>(pos) * p.ld0 + tl.n * kBlockN);
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            tmem_ld_32x32(tacc + half * 128 + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int lc = c * 4 + i;  // 16-byte chunk of this row inside the 128-column half
              int4 v = make_int4(pack_bf16(__uint_as_float(r[8 * i]) * w, __uint_as_float(r[8 * i + 1]) * w),
                                 pack_bf16(__uint_as_float(r[8 * i + 2]) * w, __uint_as_float(r[8 * i + 3]) * w),
                                 pack_bf16(__uint_as_float(r[8 * i + 4]) * w, __uint_as_float(r[8 * i + 5]) * w),
                                 pack_bf16(__uint_as_float(r[8 * i + 6]) * w, __uint_as_float(r[8 * i + 7]) * w));
              *reinterpret_cast<int4*>(stage_gen + lane * 256 + ((lc ^ (lane & 15)) << 4)) = v;
            }
          }
          __syncwarp();
          // Coalesced: 16 lanes cover one row's 256 bytes, two rows per instruction.
#pragma unroll 4
          for (int rr = 0; rr < 16; ++rr) {
            const int rsel = rr * 2 + (lane >> 4), c16 = lane & 15;
            const unsigned long long d = __shfl_sync(0xffffffffu, dst, rsel);
            const int4 v = *reinterpret_cast<const int4*>(stage_gen + rsel * 256 + ((c16 ^ (rsel & 15)) << 4));
            if (d != 0) *reinterpret_cast<int4*>(d + half * 256 + c16 * 16) = v;
          }
          __syncwarp();
        }
        if constexpr (MODE == kModeDx) {
          if (tl.n == 0 && src >= 0) {
            float dw = 0.0f;
            for (int i = 0; i < p.dwp_tiles; ++i) dw += p.dwp[static_cast<size_t>(grow) * p.dwp_tiles + i];
            p.peer_dw[src][pos] = dw;
          }
        }
        // One release per (warp, source): tells the source how many row pieces just landed.
        __syncwarp();
        for (int s = 0; s < p.lay.P; ++s) {
          const uint32_t cnt = __popc(__ballot_sync(0xffffffffu, src == s));
          if (lane == s && cnt > 0) {
            __threadfence_system();
            red_add_release_sys(p.peer_count[s], cnt);
          }
        }
      } else if constexpr (MODE == kModeDownDw) {
        const float w = valid ? p.row_w[grow] : 0.0f;
        const __nv_bfloat16* g_row = p.in0 + static_cast<size_t>(grow) * p.ld0 + tl.n * kBlockN;
        __nv_bfloat16* dy_row = p.out0 + static_cast<size_t>(grow) * p.ld0 + tl.n * kBlockN;
        float partial = 0.0f;
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          tmem_ld_32x32(tacc + c * 32, r);
          tmem_ld_wait();
          if (valid) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int4 gv = *reinterpret_cast<const int4*>(g_row + c * 32 + 8 * i);
              const uint32_t gw[4] = {static_cast<uint32_t>(gv.x), static_cast<uint32_t>(gv.y),
                                      static_cast<uint32_t>(gv.z), static_cast<uint32_t>(gv.w)};
              uint32_t o[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float g0 = bf16_lo(gw[e]), g1 = bf16_hi(gw[e]);
                // y is rounded to bf16 before the dot product, as a stored y would be.
                const uint32_t yb = pack_bf16(__uint_as_float(r[8 * i + 2 * e]), __uint_as_float(r[8 * i + 2 * e + 1]));
                partial += bf16_lo(yb) * g0 + bf16_hi(yb) * g1;
                o[e] = pack_bf16(w * g0, w * g1);
              }
              *reinterpret_cast<int4*>(dy_row + c * 32 + 8 * i) = make_int4(o[0], o[1], o[2], o[3]);
            }
          }
        }
        if (valid) p.dwp[static_cast<size_t>(grow) * p.dwp_tiles + tl.n] = partial;
      } else if constexpr (MODE == kModeDswiglu) {
        const __nv_bfloat16* h_row = p.in0 + static_cast<size_t>(grow) * p.ld0;
        __nv_bfloat16* dh_row = p.out0 + static_cast<size_t>(grow) * p.ld0;
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          const int f = tl.n * kBlockN + c * 32;
          const int b = f / p.stripe, off = f - b * p.stripe;
          const int gcol = 2 * b * p.stripe + off, ucol = gcol + p.stripe;
          tmem_ld_32x32(tacc + c * 32, r);
          tmem_ld_wait();
          if (valid) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int4 hg = *reinterpret_cast<const int4*>(h_row + gcol + 8 * i);
              const int4 hu = *reinterpret_cast<const int4*>(h_row + ucol + 8 * i);
              const uint32_t gw[4] = {static_cast<uint32_t>(hg.x), static_cast<uint32_t>(hg.y),
                                      static_cast<uint32_t>(hg.z), static_cast<uint32_t>(hg.w)};
              const uint32_t uw[4] = {static_cast<uint32_t>(hu.x), static_cast<uint32_t>(hu.y),
                                      static_cast<uint32_t>(hu.z), static_cast<uint32_t>(hu.w)};
              uint32_t og[4], ou[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                // d_act is rounded to bf16 first, as the unfused reference stores it.
                const uint32_t db = pack_bf16(__uint_as_float(r[8 * i + 2 * e]), __uint_as_float(r[8 * i + 2 * e + 1]));
                float dg[2], du[2];
#pragma unroll
                for (int z = 0; z < 2; ++z) {
                  const float d = z ? bf16_hi(db) : bf16_lo(db);
                  const float gt = z ? bf16_hi(gw[e]) : bf16_lo(gw[e]);
                  const float up = z ? bf16_hi(uw[e]) : bf16_lo(uw[e]);
                  const float sig = 1.0f / (1.0f + __expf(-gt));
                  const float sl = gt * sig;
                  dg[z] = d * up * (sig + sl * (1.0f - sig));
                  du[z] = d * sl;
                }
                og[e] = pack_bf16(dg[0], dg[1]);
                ou[e] = pack_bf16(du[0], du[1]);
              }
              *reinterpret_cast<int4*>(dh_row + gcol + 8 * i) = make_int4(og[0], og[1], og[2], og[3]);
              *reinterpret_cast<int4*>(dh_row + ucol + 8 * i) = make_int4(ou[0], ou[1], ou[2], ou[3]);
            }
          }
        }
      } else {  // kModeTgmm
        const size_t n_total = static_cast<size_t>(p.n_tiles) * kBlockN;
        const size_t m_total = static_cast<size_t>(p.m_tiles) * kBlockM;
        const size_t row_off = static_cast<size_t>(tl.m * kBlockM + row) * n_total + tl.n * kBlockN;
        const bool first = (tl.flags & kGroupFirst) != 0, final = (tl.flags & kGroupFinal) != 0;
        const float* cin = p.carry_in + row_off;
        float* cout = p.carry_out + row_off;
        auto load_chunk = [&](int col) {
          if (tl.kblocks > 0) {
            tmem_ld_32x32(tacc + col, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
          if (!first) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 pv = *reinterpret_cast<const float4*>(cin + col + 4 * i);
              r[4 * i] = __float_as_uint(__uint_as_float(r[4 * i]) + pv.x);
              r[4 * i + 1] = __float_as_uint(__uint_as_float(r[4 * i + 1]) + pv.y);
              r[4 * i + 2] = __float_as_uint(__uint_as_float(r[4 * i + 2]) + pv.z);
              r[4 * i + 3] = __float_as_uint(__uint_as_float(r[4 * i + 3]) + pv.w);
            }
          }
        };
        if (final) {
          // bf16 gradient: transpose through the warp's staging buffer so every store instruction
          // writes two full 256-byte row pieces instead of 32 scattered 16-byte ones.
          __nv_bfloat16* warp_out = p.grad_out + static_cast<size_t>(tl.g) * m_total * n_total +
                                    static_cast<size_t>(tl.m * kBlockM + q * 32) * n_total + tl.n * kBlockN;
#pragma unroll 1
          for (int half = 0; half < 2; ++half) {
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              load_chunk(half * 128 + c * 32);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int lc = c * 4 + i;
                *reinterpret_cast<int4*>(stage_gen + lane * 256 + ((lc ^ (lane & 15)) << 4)) =
                    make_int4(pack_bf16(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1])),
                              pack_bf16(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3])),
                              pack_bf16(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5])),
                              pack_bf16(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7])));
              }
            }
            __syncwarp();
#pragma unroll 4
            for (int rr = 0; rr < 16; ++rr) {
              const int rsel = rr * 2 + (lane >> 4), c16 = lane & 15;
              const int4 v = *reinterpret_cast<const int4*>(stage_gen + rsel * 256 + ((c16 ^ (rsel & 15)) << 4));
              *reinterpret_cast<int4*>(warp_out + static_cast<size_t>(rsel) * n_total + half * 128 + c16 * 8) = v;
            }
            __syncwarp();
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            load_chunk(c * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              *reinterpret_cast<float4*>(cout + c * 32 + 4 * i) =
                  make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]),
                              __uint_as_float(r[4 * i + 3]));
          }
        }
      }
      // Hand the accumulator buffer back to the MMA warp.
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(as));
    }
  }

  // ================================ teardown ================================================
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace

void launch_grouped_gemm(int mode, const GemmParams& p, const CUtensorMap& map_a, const CUtensorMap& map_b, int grid,
                         cudaStream_t stream) {
#define CEM_LAUNCH(M)                                                                                         \
  case M: {                                                                                                   \
    static bool configured = false;                                                                           \
    if (!configured) {                                                                                        \
      cudaFuncSetAttribute(grouped_gemm_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes); \
      configured = true;                                                                                      \
    }                                                                                                         \
    grouped_gemm_kernel<M><<<grid, kGemmThreads, kGemmSmemBytes, stream>>>(p, map_a, map_b);                  \
    break;                                                                                                    \
  }
  switch (mode) {
    CEM_LAUNCH(kModeSwiglu)
    CEM_LAUNCH(kModeDownFwd)
    CEM_LAUNCH(kModeDownDw)
    CEM_LAUNCH(kModeDswiglu)
    CEM_LAUNCH(kModeDx)
    CEM_LAUNCH(kModeTgmm)
    default:
      break;
  }
#undef CEM_LAUNCH
}

}  // namespace cem
