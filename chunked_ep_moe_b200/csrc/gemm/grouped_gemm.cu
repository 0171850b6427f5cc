// Grouped GEMM engine for sm_100a: persistent, warp-specialised, tcgen05 MMA with TMEM accumulators.
//
//   warp 0      TMA producer. Walks this CTA's tiles, (for the dispatch consumer) acquires the
//               arrival counters of the tile's expert, then streams A/B k-blocks into a 4-stage
//               shared-memory ring with cp.async.bulk.tensor (this CTA's shared memory only).
//   warp 1      MMA issuer. The warp walks the k-blocks in step; one elected lane issues tcgen05.mma
//               (128x256x16, bf16 -> fp32 in TMEM) and commits to the ring's empty barriers and to
//               the accumulator-full barrier.
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
#include "gemm_common.cuh"


namespace cem {

namespace {

// Issues the TMA loads of one k-block of a tile into a pipeline stage (completing on `bar`).
// (An L2 prefetch cursor running 8 k-blocks ahead of these loads was measured and made the GEMM
// modes ~14% slower at DeepSeek-V3 sizes, so there is none.)
template <int MODE>
__device__ __forceinline__ void issue_kblock(const GemmParams& p, const Tile& tl, int kb, const CUtensorMap* map_a,
                                             const CUtensorMap* map_b, uint32_t sa, uint32_t sb, uint32_t bar) {
  using Traits = ModeTraits<MODE>;
  if constexpr (Traits::kAMn) {
    // lhs [S, M]: k runs over rows; the 128-wide row tile is two 64-column chunks, one 3-D copy.
    tma_load_3d(sa, map_a, bar, tl.row0 + kb * kBlockK, tl.m * (kBlockM / 64));
  } else {
    tma_load_2d(sa, map_a, bar, kb * kBlockK, tl.row0);
  }
  if constexpr (MODE == kModeTgmm) {
    tma_load_3d(sb, map_b, bar, tl.row0 + kb * kBlockK, tl.n * (kBlockN / 64));
  } else if constexpr (Traits::kBMn) {
    // weights [L*K, N]: the 256-wide column tile is four 64-column chunks, one 3-D copy.
    tma_load_3d(sb, map_b, bar, tl.g * p.b_group_rows + kb * kBlockK, tl.n * (kBlockN / 64));
  } else {
    // weights [L*N, K] read as K-major B: 256 rows x 64 k.
    tma_load_2d(sb, map_b, bar, kb * kBlockK, tl.g * p.b_group_rows + tl.n * kBlockN);
  }
}

// Epilogue warps per CTA. Two warps per TMEM lane quarter (8 in all, each taking 128 of the 256 accumulator columns)
// were measured for the weight-gradient mode and changed nothing (0.659 vs 0.636 ms per launch at 256 experts per GPU):
// with ~256 rows per expert that mode is bound by the 22.5 GB of gradients it writes per pass, not by its epilogue.
template <int MODE>
constexpr int epilogue_warps() { return 4; }

// 168 registers per thread: 192 threads x 168 leave half of the SM's register file to a 512-thread, 64-register copy
// CTA (the dispatch put, the fp8 expansion), which has to become resident BESIDE this kernel for the overlap to happen.
template <int MODE>
__global__ void __maxnreg__(168)
grouped_gemm_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c) {
  using Traits = ModeTraits<MODE>;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzled tiles want 1024-byte aligned bases.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t staging_base = smem_base + kStages * kStageBytes;
  uint8_t* staging_gen = smem_gen + kStages * kStageBytes;
  const uint32_t bar_base = staging_base + kStagingBytes;
  // barriers: full[kStages], empty[kStages], acc_full[2], acc_empty[2], drain; then tmem slot, abort flag, early flag
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto acc_full_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };
  auto acc_empty_bar = [&](int s) { return bar_base + 8u * (2 * kStages + 2 + s); };
  const uint32_t drain_bar = bar_base + 8u * (2 * kStages + 4);
  constexpr int kSlotOff = 8 * (2 * kStages + 5);
  static_assert(kSlotOff + 12 <= kSmemTailBytes, "barrier area too small");
  const uint32_t tmem_slot = bar_base + kSlotOff;
  uint8_t* tail_gen = staging_gen + kStagingBytes;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(tail_gen + kSlotOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail_gen + kSlotOff + 4);
  volatile int* early_flag = reinterpret_cast<volatile int*>(tail_gen + kSlotOff + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool counting = p.prof != nullptr;
  auto prof_add = [&](int slot, long long v) {
    atomicAdd(p.prof + static_cast<size_t>(blockIdx.x) * kProfSlots + slot, static_cast<unsigned long long>(v));
  };

  // The aligned layout must fit into what the launch provided (the slack covers a base that is not 1024-byte aligned).
  if (smem_base - smem_u32(smem_raw) > static_cast<uint32_t>(kSmemAlignSlack)) {
    if (threadIdx.x == 0) report_status(p.status, kStatusBadIndex, kKernelGemm, MODE, -1, 0, kSmemAlignSlack,
                                        smem_base - smem_u32(smem_raw));
    return;
  }
  // An earlier kernel of this pass already gave up: do nothing, so the error reaches the host quickly.
  if (threadIdx.x == 0) *early_flag = (p.status != nullptr && p.status->code != 0) ? 1 : 0;
  __syncthreads();
  if (*early_flag) return;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(acc_full_bar(s), 1);
      mbar_init(acc_empty_bar(s), epilogue_warps<MODE>());
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if constexpr (MODE == kModeTgmm) tma_prefetch_desc(&map_c);
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
    long long empty_wait = 0;
    {
      // The whole warp walks the k-blocks in step (every lane waits on the stage's barrier, one elected lane issues
      // the copies), so stage index, phase and addresses stay warp-uniform values.
      uint32_t ps = 0, pph = 0;
      bool dead = false;
      // The next tile is decoded one iteration ahead, so its plan-table load is in flight while this tile runs.
      Tile nxt = {};
      if (blockIdx.x < num_tiles) nxt = decode_tile<MODE>(p, blockIdx.x, num_entries);
      for (int t = blockIdx.x; t < num_tiles && !dead && !*abort_flag; t += gridDim.x) {
        const Tile tl = nxt;
        if (t + static_cast<int>(gridDim.x) < num_tiles) nxt = decode_tile<MODE>(p, t + static_cast<int>(gridDim.x), num_entries);
        if constexpr (MODE == kModeSwiglu) {
          if ((p.arrive != nullptr || p.ready != nullptr) && tl.g != waited_expert) {
            if (!wait_expert_rows(p, tl.g, lane, abort_flag)) break;
            waited_expert = tl.g;
          }
        }
        for (int kb = 0; kb < tl.kblocks; ++kb) {
          const long long w0 = counting ? clock64() : 0;
          bool ok = mbar_wait(empty_bar(ps), pph ^ 1u, p.mbar_limit, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) {
            if (lane == 0) {
              report_status(p.status, kStatusMbarTimeout, kKernelGemm, MODE, t, 100 + ps, 0, 0);
              *abort_flag = 1;
            }
            dead = true;
            break;
          }
          if (counting) empty_wait += clock64() - w0;
          if (elect_one()) {
            const uint32_t sa = smem_base + ps * kStageBytes;
            mbar_expect_tx(full_bar(ps), kStageBytes);
            issue_kblock<MODE>(p, tl, kb, &map_a, &map_b, sa, sa + kStageBytesA, full_bar(ps));
          }
          ++it;
          if (++ps == kStages) { ps = 0; pph ^= 1u; }
        }
      }
      __syncwarp();
    }
    if (counting && lane == 0) prof_add(kProfEmptyWait, empty_wait);
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
    // All 32 lanes run the loop together (waits included) and ONE elected lane issues; loop counters, stage
    // addresses and descriptors are then warp-uniform values. A loop run by a single lane inside a divergent branch
    // cost ~610-780 cycles per k-block in this kernel and ~640-925 in the CTA-pair kernel; this form measures
    // ~610-700 and ~520-630 (the tensor pipe's floor is 512).
    constexpr uint32_t idesc = make_instr_desc_bf16(kBlockM, kBlockN, Traits::kAMn, Traits::kBMn);
    constexpr uint32_t kDescStepA = Traits::kAMn ? 2048u : 32u;  // bytes per 16-wide k step inside a stage
    constexpr uint32_t kDescStepB = Traits::kBMn ? 2048u : 32u;
    uint32_t it = 0, tcount = 0;
    long long full_wait = 0, acc_wait = 0;
    const long long loop_c0 = counting ? clock64() : 0;
    const uint64_t loop_n0 = counting ? global_timer_ns() : 0;
    {
      // The whole warp walks the k-blocks in step: every lane waits on the stage's barrier, one elected lane (always
      // the same one) issues the four MMAs and the commit. Stage index, phase and descriptors are warp-uniform values
      // computed outside any divergent region.
      uint32_t cs = 0, cph = 0;
      bool dead = false;
      auto issue_stage = [&](uint32_t s, uint32_t tmem_d, int ksteps, bool first_kblock) {
        const uint32_t sa = smem_base + s * kStageBytes;
        const uint64_t da = Traits::kAMn ? make_smem_desc(sa, 8192, 1024) : make_smem_desc(sa, 16, 1024);
        const uint64_t db = Traits::kBMn ? make_smem_desc(sa + kStageBytesA, 8192, 1024)
                                         : make_smem_desc(sa + kStageBytesA, 16, 1024);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            // The start address sits in the low 14 bits (16-byte units) and never carries out of them.
            if (k < ksteps)
              umma_bf16(tmem_d, da + ((k * kDescStepA) >> 4), db + ((k * kDescStepB) >> 4), idesc,
                        (!first_kblock || k > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(s));
        }
      };
      auto fail = [&](int t, int detail) {
        if (lane == 0) {
          report_status(p.status, kStatusMbarTimeout, kKernelGemm, MODE, t, detail, 0, 0);
          *abort_flag = 1;
        }
        dead = true;
      };
      // The next tile is decoded one iteration ahead, so its plan-table load is in flight while this tile runs.
      Tile nxt = {};
      if (blockIdx.x < num_tiles) nxt = decode_tile<MODE>(p, blockIdx.x, num_entries);
      for (int t = blockIdx.x; t < num_tiles && !dead && !*abort_flag; t += gridDim.x, ++tcount) {
        const Tile tl = nxt;
        if (t + static_cast<int>(gridDim.x) < num_tiles) nxt = decode_tile<MODE>(p, t + static_cast<int>(gridDim.x), num_entries);
        const int as = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1u;
        const uint32_t tmem_d = tmem_base + as * kBlockN;
        // Weight gradients: the last k-block of a group may hold rows of the next group.
        const bool ragged_tail = (MODE == kModeTgmm) && (tl.nrows % kBlockK) != 0;
        const int solo_kblocks = ragged_tail ? tl.kblocks - 1 : tl.kblocks;
        const long long w0 = counting ? clock64() : 0;
        bool ok = __all_sync(0xffffffffu, mbar_wait(acc_empty_bar(as), aph ^ 1u, p.mbar_limit, abort_flag));
        if (counting) acc_wait += clock64() - w0;
        if (!ok) { fail(t, 200 + as); break; }
        tcgen05_fence_after_sync();
        for (int kb = 0; kb < solo_kblocks; ++kb) {
          const long long w1 = counting ? clock64() : 0;
          ok = __all_sync(0xffffffffu, mbar_wait(full_bar(cs), cph, p.mbar_limit, abort_flag));
          if (counting) full_wait += clock64() - w1;
          if (!ok) { fail(t, 300 + cs); break; }
          tcgen05_fence_after_sync();
          issue_stage(cs, tmem_d, kBlockK / kUmmaK, kb == 0);
          ++it;
          if (++cs == kStages) { cs = 0; cph ^= 1u; }
        }
        if (dead) break;
        if constexpr (MODE == kModeTgmm) {
          if (ragged_tail) {
            const int kb = tl.kblocks - 1;
            const long long w1 = counting ? clock64() : 0;
            ok = __all_sync(0xffffffffu, mbar_wait(full_bar(cs), cph, p.mbar_limit, abort_flag));
            if (counting) full_wait += clock64() - w1;
            if (!ok) { fail(t, 300 + cs); break; }
            const int valid = tl.nrows - kb * kBlockK;  // rows of this k-block inside the group
            const int ksteps = (valid + kUmmaK - 1) / kUmmaK;
            // Rows [valid, ksteps*16) belong to the next group (or are padding): zero them in both operands.
            // A k row is one 128-byte line per 64-column chunk, 48 16-byte pieces in all (6 chunks x 8): lane i clears
            // piece i of chunks 0-3, lanes 0-15 also piece 32+i of chunks 4-5.
            uint8_t* ga = smem_gen + cs * kStageBytes;
            const int zrows = ksteps * kUmmaK - valid;
            uint8_t* lo = ga + (lane >> 3) * 8192 + (lane & 7) * 16 + valid * 128;
            uint8_t* hi = lo + 4 * 8192;
            for (int r = 0; r < zrows; ++r, lo += 128, hi += 128) {
              *reinterpret_cast<int4*>(lo) = make_int4(0, 0, 0, 0);
              if (lane < 16) *reinterpret_cast<int4*>(hi) = make_int4(0, 0, 0, 0);
            }
            fence_proxy_async_smem();
            __syncwarp();
            tcgen05_fence_after_sync();
            issue_stage(cs, tmem_d, ksteps, kb == 0);
            ++it;
            if (++cs == kStages) { cs = 0; cph ^= 1u; }
          }
        }
        if (elect_one()) {
          if (tl.kblocks > 0) {
            umma_commit(acc_full_bar(as));
          } else {
            mbar_arrive(acc_full_bar(as));  // empty group: nothing was issued, the epilogue writes zeros
          }
        }
      }
      __syncwarp();
    }
    if (counting && lane == 0) {
      prof_add(kProfLoopCycles, clock64() - loop_c0);
      prof_add(kProfLoopNs, static_cast<long long>(global_timer_ns() - loop_n0));
      prof_add(kProfFullWait, full_wait);
      prof_add(kProfAccWait, acc_wait);
      prof_add(kProfKBlocks, it);
      prof_add(kProfTiles, tcount);
    }
    if (*abort_flag) {
      // Unwinding: let the MMAs already issued finish before TMEM is freed (the commit comes from the elected lane,
      // which issued them).
      __syncwarp();
      if (elect_one()) umma_commit(drain_bar);
      mbar_wait(drain_bar, 0, p.mbar_limit);
    }
  } else {
    // ================================ epilogue ==============================================
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    const int ew = warp - 2;             // epilogue warp index
    constexpr int kColsPerWarp = kBlockN * 4 / epilogue_warps<MODE>();  // warps sharing a lane quarter split the columns
    const int col0 = (ew >> 2) * kColsPerWarp;
    const int ncols = kColsPerWarp;
    // Weight gradients stage swizzled 4 KB blocks for tiled TMA stores (1024-byte aligned, 8 KB per warp); every other
    // mode stages padded rows.
    uint8_t* stage_gen = staging_gen + ew * (MODE == kModeTgmm ? 8192 : kStagingBytes / epilogue_warps<MODE>());
    uint32_t tcount = 0, returned = 0;
    long long epi_wait = 0;
    // The next tile is decoded one iteration ahead, so its plan-table load is in flight while this tile runs.
    Tile nxt = {};
    if (blockIdx.x < num_tiles) nxt = decode_tile<MODE>(p, blockIdx.x, num_entries);
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x, ++tcount) {
      const Tile tl = nxt;
      if (t + static_cast<int>(gridDim.x) < num_tiles) nxt = decode_tile<MODE>(p, t + static_cast<int>(gridDim.x), num_entries);
      prefetch_epilogue_inputs<MODE>(p, tl, warp & 3, lane);
      const int as = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1u;
      const long long w0 = counting ? clock64() : 0;
      bool ok = mbar_wait(acc_full_bar(as), aph, p.mbar_limit, abort_flag);
      if (counting) epi_wait += clock64() - w0;
      if (!ok) {
        report_status(p.status, kStatusMbarTimeout, kKernelGemm, MODE, t, 400 + as, 0, 0);
        *abort_flag = 1;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after_sync();
      const uint32_t tacc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * kBlockN;
      run_epilogue<MODE>(p, tl, tacc, q, lane, stage_gen, returned, &map_c, col0, ncols);
      // Hand the accumulator buffer back to the MMA warp.
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(as));
    }
    if (counting && ew == 0 && lane == 0) prof_add(kProfEpiWait, epi_wait);
    if constexpr (Traits::kCombine) flush_returned(p, lane, returned);  // also on the unwind path: what was stored is released
    else bulk_wait_all();  // bulk stores of this thread still read the staging rows: no exit before they are done
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

int g_gemm_extra_smem = 0;

void launch_grouped_gemm(int mode, const GemmParams& p, const CUtensorMap& map_a, const CUtensorMap& map_b,
                         const CUtensorMap& map_c, int grid, cudaStream_t stream) {
#define CEM_LAUNCH(M)                                                                                         \
  case M: {                                                                                                   \
    static bool configured = false;                                                                           \
    if (!configured) {                                                                                        \
      cudaFuncSetAttribute(grouped_gemm_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes + 1024); \
      configured = true;                                                                                      \
    }                                                                                                         \
    grouped_gemm_kernel<M><<<grid, 64 + 32 * epilogue_warps<M>(), kGemmSmemBytes + g_gemm_extra_smem, stream>>>(    \
        p, map_a, map_b, map_c);                                                                              \
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
