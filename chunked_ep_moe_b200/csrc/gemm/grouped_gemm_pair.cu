// CTA-pair variant of the grouped GEMM engine: two CTAs of one cluster drive ONE 256 x 256 x 16
// tcgen05.mma (cta_group::2). Each CTA stages only its own 128 rows of A and its own 128 columns
// of B (32 KB per k-block instead of 48 KB), which is what lifts the single-CTA kernel's shared-memory
// bandwidth bound and allows a 6-stage ring in the same 192 KB.
//
//   both CTAs   warp 0      TMA producer for the CTA's own A rows / B half, completing on the CTA's own
//                           full barrier (plain CTA-local loads).
//   leader      warp 1      waits for its own stage AND the peer's "stage ready" arrival, issues the pair
//                           MMAs, commits to both CTAs' empty barriers and both accumulator-full barriers.
//   peer        warp 1      weight-gradient mode only: for a tile's ragged last k-block it waits for its own
//                           loads, zero-fills the rows past the group and forwards the arrival to the leader.
//   both CTAs   warps 2-5   epilogue of the CTA's own 128 x 256 accumulator half (same code as the
//                           single-CTA kernel), then arrive on the leader's accumulator-empty barrier.
//
// A pair covers two consecutive 128-row tiles of ONE expert (they share its weights); an odd last tile is
// a pair whose second half stores nothing. In the weight-gradient mode the pair splits the dense feature
// dimension instead. Every wait is bounded; a CTA that gives up records a status and unwinds, and its
// partner then runs into its own limits.
#include "gemm_common.cuh"

namespace cem {

namespace {

constexpr int kPairStages = 6;
constexpr int kPairStageBytesA = kBlockM * kBlockK * 2;        // 16 KB: this CTA's 128 rows
constexpr int kPairStageBytesB = (kBlockN / 2) * kBlockK * 2;  // 16 KB: this CTA's 128 columns
constexpr int kPairStageBytes = kPairStageBytesA + kPairStageBytesB;
constexpr int kPairBand = kRasterBand / 2;                     // pairs swept together across N

// Wait on a barrier that the partner CTA (its MMA commits, its relay warp) completes: polled or suspending.
__device__ __forceinline__ bool pair_wait(int suspend, uint32_t bar, uint32_t parity, uint32_t limit_us,
                                          const volatile int* abort = nullptr) {
  return suspend ? mbar_wait(bar, parity, limit_us, abort) : mbar_wait_poll(bar, parity, limit_us, abort);
}

// Tile as seen by CTA `rank` of the pair.
template <int MODE>
__device__ __forceinline__ Tile decode_pair_tile(const GemmParams& p, int t, int num_entries, int rank) {
  Tile tl;
  if constexpr (MODE == kModeTgmm) {
    const int m_pairs = p.m_tiles / 2;
    const int per_group = m_pairs * p.n_tiles;
    const int gi = t / per_group, rem = t - gi * per_group;
    const int4 e = reinterpret_cast<const int4*>(p.plan + p.lay.off_gtiles + 4 * p.lay.max_gtiles * p.slice)[gi];
    tl.g = e.x; tl.row0 = e.y; tl.nrows = e.z; tl.flags = e.w;
    const int mp = rem / p.n_tiles;
    tl.m = 2 * mp + rank; tl.n = rem - mp * p.n_tiles;
    tl.kblocks = (e.z + kBlockK - 1) / kBlockK;
  } else {
    const int band_tiles = kPairBand * p.n_tiles;
    const int band = t / band_tiles, rem = t - band * band_tiles;
    int width = num_entries - band * kPairBand;
    width = width > kPairBand ? kPairBand : width;
    tl.n = rem / width;
    const int pi = band * kPairBand + (rem - tl.n * width);
    const int4 e = reinterpret_cast<const int4*>(p.plan + p.lay.off_ptiles + 4 * p.lay.max_ptiles * p.slice)[pi];
    tl.g = e.x;
    tl.row0 = e.y + rank * kBlockM;
    tl.nrows = plan_clip(e.z - rank * kBlockM, 0, kBlockM);
    tl.flags = 0; tl.m = pi;
    tl.kblocks = p.k_blocks;
  }
  return tl;
}

// `bar` is the LEADER's full barrier (pair-aware loads credit the leader directly), except for `direct == false`
// (the peer's ragged last k-block in the weight-gradient mode): then it is this CTA's own full barrier and the loads
// are plain ones.
template <int MODE>
__device__ __forceinline__ void issue_pair_kblock(const GemmParams& p, const Tile& tl, int kb, int rank,
                                                  const CUtensorMap* map_a, const CUtensorMap* map_b, uint32_t sa,
                                                  uint32_t sb, uint32_t bar, bool direct) {
  using Traits = ModeTraits<MODE>;
  const int chunk0 = tl.n * (kBlockN / 64) + rank * (kBlockN / 128);  // this CTA's half of the 256-wide column tile
  if constexpr (MODE == kModeTgmm) {
    // A and B are both two 64-column chunks
    if (direct) {
      tma_load_3d_pair(sa, map_a, bar, tl.row0 + kb * kBlockK, tl.m * (kBlockM / 64));
      tma_load_3d_pair(sb, map_b, bar, tl.row0 + kb * kBlockK, chunk0);
    } else {
      tma_load_3d(sa, map_a, bar, tl.row0 + kb * kBlockK, tl.m * (kBlockM / 64));
      tma_load_3d(sb, map_b, bar, tl.row0 + kb * kBlockK, chunk0);
    }
  } else {
    tma_load_2d_pair(sa, map_a, bar, kb * kBlockK, tl.row0);
    if constexpr (Traits::kBMn) {
      tma_load_3d_pair(sb, map_b, bar, tl.g * p.b_group_rows + kb * kBlockK, chunk0);
    } else {
      tma_load_2d_pair(sb, map_b, bar, kb * kBlockK, tl.g * p.b_group_rows + tl.n * kBlockN + rank * (kBlockN / 2));  // 128-row box
    }
  }
}

// 168 registers per thread: 192 threads x 168 leave half of the SM's register file to a 512-thread, 64-register copy
// CTA (the dispatch put, the fp8 expansion), which has to become resident BESIDE this kernel for the overlap to happen.
template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __maxnreg__(168)
grouped_gemm_pair_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ CUtensorMap map_a,
                         const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c) {
  using Traits = ModeTraits<MODE>;
  // Every load credits the leader's full barrier directly, with one exception: the last k-block of a weight-gradient
  // tile whose group does not end on a 64-row boundary needs rows zeroed by the CTA that owns them BEFORE the leader
  // may use them. For that k-block the peer loads onto its own full barrier, its warp 1 zero-fills and then makes the
  // arrival on the leader's barrier that the peer's producer makes for every other k-block. (An earlier form relayed
  // EVERY k-block of that mode through the peer's warp 1: one more hop on the critical path of each stage.)
  constexpr bool kRelay = (MODE == kModeTgmm);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t staging_base = smem_base + kPairStages * kPairStageBytes;
  uint8_t* staging_gen = smem_gen + kPairStages * kPairStageBytes;
  const uint32_t bar_base = staging_base + kStagingBytes;
  // barriers: full[6], empty[6], peer_ready[6], acc_full[2], acc_empty[2], drain; then tmem slot, abort flag
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kPairStages + s); };
  auto ready_bar = [&](int s) { return bar_base + 8u * (2 * kPairStages + s); };
  auto acc_full_bar = [&](int s) { return bar_base + 8u * (3 * kPairStages + s); };
  auto acc_empty_bar = [&](int s) { return bar_base + 8u * (3 * kPairStages + 2 + s); };
  const uint32_t drain_bar = bar_base + 8u * (3 * kPairStages + 4);
  constexpr int kSlotOff = 8 * (3 * kPairStages + 5);
  static_assert(kSlotOff + 12 <= kSmemTailBytes, "barrier area too small");
  const uint32_t tmem_slot = bar_base + kSlotOff;
  uint8_t* tail_gen = staging_gen + kStagingBytes;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(tail_gen + kSlotOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail_gen + kSlotOff + 4);
  volatile int* early_flag = reinterpret_cast<volatile int*>(tail_gen + kSlotOff + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_cta_rank());
  const bool leader = rank == 0;
  const bool counting = p.prof != nullptr;
  auto prof_add = [&](int slot, long long v) {
    atomicAdd(p.prof + static_cast<size_t>(blockIdx.x) * kProfSlots + slot, static_cast<unsigned long long>(v));
  };

  // A CTA that gives up tells its partner too (the flag sits at the same offset in both CTAs), so the partner's waits
  // end at their next poll instead of running into their own limits.
  const uint32_t partner_abort = map_to_cta(bar_base + kSlotOff + 4, static_cast<uint32_t>(rank ^ 1));
  auto raise_abort = [&]() {
    *abort_flag = 1;
    st_shared_cluster_u32(partner_abort, 1u);
  };

  // The aligned layout must fit into what the launch provided. Both CTAs of a pair see the same offsets, so they
  // leave together.
  if (smem_base - smem_u32(smem_raw) > static_cast<uint32_t>(kSmemAlignSlack)) {
    if (threadIdx.x == 0) report_status(p.status, kStatusBadIndex, kKernelGemm, MODE, -1, 1, kSmemAlignSlack,
                                        smem_base - smem_u32(smem_raw));
    return;
  }
  // An earlier kernel of this pass already gave up: both CTAs of the pair leave together (the leader decides).
  if (threadIdx.x == 0 && leader) {
    const uint32_t v = (p.status != nullptr && p.status->code != 0) ? 1u : 0u;
    *early_flag = static_cast<int>(v);
    st_shared_cluster_u32(map_to_cta(bar_base + kSlotOff + 8, 1), v);
  }
  cluster_sync_all();
  if (*early_flag) return;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      // leader: one arrival from each CTA of the pair; the peer's own barrier only sees its ragged-tail loads
      mbar_init(full_bar(s), (kRelay && !leader) ? 1 : 2);
      mbar_init(empty_bar(s), 1);
      mbar_init(ready_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(acc_full_bar(s), 1);
      mbar_init(acc_empty_bar(s), 8);  // four epilogue warps in each CTA of the pair
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if constexpr (MODE == kModeTgmm) tma_prefetch_desc(&map_c);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anyone signals across the pair
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;

  const int num_entries = (MODE == kModeTgmm) ? p.plan[p.lay.off_num_gtiles + p.slice]
                                              : p.plan[p.lay.off_num_ptiles + p.slice];
  const int num_tiles = (MODE == kModeTgmm) ? num_entries * (p.m_tiles / 2) * p.n_tiles : num_entries * p.n_tiles;
  const int first_tile = blockIdx.x >> 1, tile_step = gridDim.x >> 1;

  if (warp == 0) {
    // ================================ TMA producer (both CTAs) ==============================
    uint32_t it = 0;
    uint32_t own_used = 0, own_parity = 0;  // per stage: this CTA's own full barrier has been used / parity of its next use
    int waited_expert = -1;
    long long empty_wait = 0;
    {
      // The whole warp walks the k-blocks in step; one elected lane issues the copies.
      uint32_t ps = 0, pph = 0;
      bool dead = false;
      // The next tile is decoded one iteration ahead, so its plan-table load is in flight while this tile runs.
      Tile nxt = {};
      if (first_tile < num_tiles) nxt = decode_pair_tile<MODE>(p, first_tile, num_entries, rank);
      for (int t = first_tile; t < num_tiles && !dead && !*abort_flag; t += tile_step) {
        const Tile tl = nxt;
        if (t + tile_step < num_tiles) nxt = decode_pair_tile<MODE>(p, t + tile_step, num_entries, rank);
        if constexpr (MODE == kModeSwiglu) {
          if ((p.arrive != nullptr || p.ready != nullptr) && tl.g != waited_expert) {
            if (!wait_expert_rows(p, tl.g, lane, abort_flag)) {
              if (lane == 0) raise_abort();
              break;
            }
            waited_expert = tl.g;
          }
        }
        for (int kb = 0; kb < tl.kblocks; ++kb) {
          const long long w0 = counting ? clock64() : 0;
          const bool ok = __all_sync(0xffffffffu, pair_wait(p.suspend_waits, empty_bar(ps), pph ^ 1u, p.mbar_limit, abort_flag));
          if (!ok) {
            if (lane == 0) {
              report_status(p.status, kStatusMbarTimeout, kKernelGemm, MODE, t, 1100 + ps, 0, 0);
              raise_abort();
            }
            dead = true;
            break;
          }
          if (counting) empty_wait += clock64() - w0;
          const bool own = kRelay && !leader && kb == tl.kblocks - 1 && (tl.nrows % kBlockK) != 0;
          if (own) {
            own_used |= 1u << ps;
            own_parity ^= 1u << ps;
          }
          if (elect_one()) {
            const uint32_t sa = smem_base + ps * kPairStageBytes;
            const uint32_t fb = own ? full_bar(ps) : map_to_cta(full_bar(ps), 0);
            if (own) mbar_expect_tx(fb, kPairStageBytes); else mbar_expect_tx_cluster(fb, kPairStageBytes);
            issue_pair_kblock<MODE>(p, tl, kb, rank, &map_a, &map_b, sa, sa + kPairStageBytesA, fb, !own);
          }
          ++it;
          if (++ps == kPairStages) { ps = 0; pph ^= 1u; }
        }
      }
      __syncwarp();
    }
    if (counting && lane == 0) prof_add(kProfEmptyWait, empty_wait);
    // Unwinding: no exit while a copy may still land in this CTA's shared memory. The leader's barriers see every
    // stage of both CTAs; the peer's own barriers only its ragged-tail loads (their last use has the parity before
    // the next one's).
    if (lane == 0 && *abort_flag) {
      for (int s = 0; s < kPairStages; ++s) {
        if (leader) {
          if (it > static_cast<uint32_t>(s)) {
            const uint32_t last = it - 1 - ((it - 1 - s) % kPairStages);
            mbar_wait(full_bar(s), (last / kPairStages) & 1u, p.mbar_limit);
          }
        } else if ((own_used >> s) & 1u) {
          mbar_wait(full_bar(s), ((own_parity >> s) & 1u) ^ 1u, p.mbar_limit);
        }
      }
    }
  } else if (warp == 1) {
    // ================================ MMA issuer (leader) / stage relay (peer) ==============
    // As in the single-CTA kernel, the whole warp walks the k-blocks in step and one elected lane issues.
    constexpr uint32_t idesc = make_instr_desc_bf16(2 * kBlockM, kBlockN, Traits::kAMn, Traits::kBMn);
    constexpr uint32_t kDescStepA = Traits::kAMn ? 2048u : 32u;
    constexpr uint32_t kDescStepB = Traits::kBMn ? 2048u : 32u;
    const uint32_t peer = static_cast<uint32_t>(rank ^ 1);
    uint32_t it = 0, tcount = 0;
    uint32_t own_phase = 0;  // peer, weight-gradient mode: parity of the next use of its own full barrier, per stage
    long long full_wait = 0, acc_wait = 0;
    const long long loop_c0 = counting ? clock64() : 0;
    const uint64_t loop_n0 = counting ? global_timer_ns() : 0;
    {
      // The whole warp walks the k-blocks in step; one elected lane (always the same one) issues MMAs and commits.
      uint32_t cs = 0, cph = 0;
      bool dead = false;
      auto issue_stage = [&](uint32_t s, uint32_t tmem_d, int ksteps, bool first_kblock) {
        const uint32_t sa = smem_base + s * kPairStageBytes;
        const uint64_t da = Traits::kAMn ? make_smem_desc(sa, 8192, 1024) : make_smem_desc(sa, 16, 1024);
        const uint64_t db = Traits::kBMn ? make_smem_desc(sa + kPairStageBytesA, 8192, 1024)
                                         : make_smem_desc(sa + kPairStageBytesA, 16, 1024);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            if (k < ksteps)
              umma_bf16_pair(tmem_d, da + ((k * kDescStepA) >> 4), db + ((k * kDescStepB) >> 4), idesc,
                             (!first_kblock || k > 0) ? 1u : 0u);
          }
          umma_commit_pair_both(empty_bar(s));
        }
      };
      auto fail = [&](int t, int detail) {
        if (lane == 0) {
          report_status(p.status, kStatusMbarTimeout, kKernelGemm, MODE, t, detail, 0, 0);
          raise_abort();
        }
        dead = true;
      };
      auto advance = [&]() {
        ++it;
        if (++cs == kPairStages) { cs = 0; cph ^= 1u; }
      };
      // The next tile is decoded one iteration ahead, so its plan-table load is in flight while this tile runs.
      Tile nxt = {};
      if (first_tile < num_tiles) nxt = decode_pair_tile<MODE>(p, first_tile, num_entries, rank);
      for (int t = first_tile; t < num_tiles && !dead && !*abort_flag && (kRelay || leader); t += tile_step, ++tcount) {
        const Tile tl = nxt;
        if (t + tile_step < num_tiles) nxt = decode_pair_tile<MODE>(p, t + tile_step, num_entries, rank);
        const int as = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1u;
        const uint32_t tmem_d = tmem_base + as * kBlockN;
        const bool ragged_tail = kRelay && (tl.nrows % kBlockK) != 0;
        const int solo_kblocks = ragged_tail ? tl.kblocks - 1 : tl.kblocks;
        bool ok = true;
        if (leader) {
          const long long w0 = counting ? clock64() : 0;
          ok = __all_sync(0xffffffffu, pair_wait(p.suspend_waits, acc_empty_bar(as), aph ^ 1u, p.mbar_limit, abort_flag));
          if (counting) acc_wait += clock64() - w0;
          if (!ok) { fail(t, 1200 + as); break; }
          tcgen05_fence_after_sync();
        }
        for (int kb = 0; kb < solo_kblocks; ++kb) {
          if (leader) {
            const long long w1 = counting ? clock64() : 0;
            ok = __all_sync(0xffffffffu, mbar_wait(full_bar(cs), cph, p.mbar_limit, abort_flag));
            if (counting) full_wait += clock64() - w1;
            if (!ok) { fail(t, 1300 + cs); break; }
            tcgen05_fence_after_sync();
            issue_stage(cs, tmem_d, kBlockK / kUmmaK, kb == 0);
          }
          advance();  // the peer only keeps count of the stages: its loads credit the leader's barrier
        }
        if (dead) break;
        if constexpr (kRelay) {
          if (ragged_tail) {
            const int kb = tl.kblocks - 1;
            // Leader: both halves have landed and the peer has zero-filled its rows. Peer: its own loads have landed.
            const uint32_t parity = leader ? cph : ((own_phase >> cs) & 1u);
            own_phase ^= 1u << cs;
            ok = __all_sync(0xffffffffu, mbar_wait(full_bar(cs), parity, p.mbar_limit, abort_flag));
            if (!ok) { fail(t, 1300 + cs); break; }
            const int valid = tl.nrows - kb * kBlockK;
            const int ksteps = (valid + kUmmaK - 1) / kUmmaK;
            // Zero this CTA's rows [valid, ksteps*16) in its four 64-column chunks (2 of A, 2 of B): a k row is 32
            // 16-byte pieces here, lane i clears piece i.
            uint8_t* ga = smem_gen + cs * kPairStageBytes;
            const int zrows = ksteps * kUmmaK - valid;
            uint8_t* piece = ga + (lane >> 3) * 8192 + (lane & 7) * 16 + valid * 128;
            for (int r = 0; r < zrows; ++r, piece += 128) *reinterpret_cast<int4*>(piece) = make_int4(0, 0, 0, 0);
            fence_proxy_async_smem();
            __syncwarp();
            if (!leader) {
              // the arrival the peer's producer makes for every other k-block, after the rows are clean
              if (elect_one()) mbar_arrive_cluster(map_to_cta(full_bar(cs), peer));
            } else {
              tcgen05_fence_after_sync();
              issue_stage(cs, tmem_d, ksteps, kb == 0);
            }
            advance();
          }
        }
        if (leader && elect_one()) {
          if (tl.kblocks > 0) {
            umma_commit_pair_both(acc_full_bar(as));
          } else {
            mbar_arrive(acc_full_bar(as));  // empty group: both epilogues write zeros
            mbar_arrive_cluster(map_to_cta(acc_full_bar(as), peer));
          }
        }
      }
      __syncwarp();
    }
    if (counting && leader && lane == 0) {
      prof_add(kProfLoopCycles, clock64() - loop_c0);
      prof_add(kProfLoopNs, static_cast<long long>(global_timer_ns() - loop_n0));
      prof_add(kProfFullWait, full_wait);
      prof_add(kProfAccWait, acc_wait);
      prof_add(kProfKBlocks, it);
      prof_add(kProfTiles, tcount);
    }
    if (leader && *abort_flag) {
      __syncwarp();
      if (elect_one()) umma_commit_pair(drain_bar);
      mbar_wait(drain_bar, 0, p.mbar_limit);
    }
  } else {
    // ================================ epilogue (both CTAs) ==================================
    const int q = warp & 3;
    uint8_t* stage_gen = staging_gen + (warp - 2) * (MODE == kModeTgmm ? 8192 : kStagingBytes / 4);
    const uint32_t leader_acc_empty0 = map_to_cta(acc_empty_bar(0), 0);
    uint32_t tcount = 0, returned = 0;
    // The next tile is decoded one iteration ahead, so its plan-table load is in flight while this tile runs.
    Tile nxt = {};
    if (first_tile < num_tiles) nxt = decode_pair_tile<MODE>(p, first_tile, num_entries, rank);
    for (int t = first_tile; t < num_tiles && !*abort_flag; t += tile_step, ++tcount) {
      const Tile tl = nxt;
      if (t + tile_step < num_tiles) nxt = decode_pair_tile<MODE>(p, t + tile_step, num_entries, rank);
      prefetch_epilogue_inputs<MODE>(p, tl, warp & 3, lane);
      const int as = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1u;
      bool ok = pair_wait(p.suspend_waits, acc_full_bar(as), aph, p.mbar_limit, abort_flag);
      if (!ok) {
        report_status(p.status, kStatusMbarTimeout, kKernelGemm, MODE, t, 1500 + as, 0, 0);
        raise_abort();
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after_sync();
      const uint32_t tacc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * kBlockN;
      run_epilogue<MODE>(p, tl, tacc, q, lane, stage_gen, returned, &map_c);
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_acc_empty0 + 8u * as);
    }
    if constexpr (Traits::kCombine) flush_returned(p, lane, returned);  // also on the unwind path: what was stored is released
    else bulk_wait_all();  // bulk stores of this thread still read the staging rows: no exit before they are done
  }

  // ================================ teardown ================================================
  tcgen05_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // nobody frees TMEM or leaves while its partner may still signal or compute
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// Largest persistent grid whose clusters are all resident at once. A cluster needs both SMs of one TPC free,
// so this can be fewer than SM-count / 2 clusters; a cluster that does not fit would only start after the first
// wave has finished ALL of its (statically assigned) tiles and double the kernel's time.
template <typename Kernel>
int resident_pair_grid(Kernel kernel, int requested) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(requested), 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = kGemmSmemBytes + g_gemm_extra_smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess || clusters <= 0) {
    cudaGetLastError();
    return requested;
  }
  const int grid = 2 * clusters;
  return grid < requested ? grid : requested;
}

}  // namespace

int g_pair_grid_used = 0;  // last pair grid size, for diagnostics
int g_pair_suspend_waits = 0;

void launch_grouped_gemm_pair(int mode, const GemmParams& p_in, const CUtensorMap& map_a, const CUtensorMap& map_b,
                              const CUtensorMap& map_c, int grid, cudaStream_t stream) {
  GemmParams p = p_in;
  p.suspend_waits = g_pair_suspend_waits;
  grid &= ~1;  // whole pairs only
#define CEM_LAUNCH_PAIR(M)                                                                                       \
  case M: {                                                                                                      \
    static int resident = 0;                                                                                     \
    if (resident == 0) {                                                                                         \
      cudaFuncSetAttribute(grouped_gemm_pair_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize,             \
                           kGemmSmemBytes + 1024);                                                               \
      resident = resident_pair_grid(grouped_gemm_pair_kernel<M>, grid);                                          \
    }                                                                                                            \
    const int g = grid < resident ? grid : resident;                                                             \
    g_pair_grid_used = g;                                                                                        \
    grouped_gemm_pair_kernel<M><<<g, kGemmThreads, kGemmSmemBytes + g_gemm_extra_smem, stream>>>(p, map_a, map_b,      \
                                                                                                  map_c);        \
    break;                                                                                                       \
  }
  switch (mode) {
    CEM_LAUNCH_PAIR(kModeSwiglu)
    CEM_LAUNCH_PAIR(kModeDownFwd)
    CEM_LAUNCH_PAIR(kModeDownDw)
    CEM_LAUNCH_PAIR(kModeDswiglu)
    CEM_LAUNCH_PAIR(kModeDx)
    CEM_LAUNCH_PAIR(kModeTgmm)
    default:
      break;
  }
#undef CEM_LAUNCH_PAIR
}

}  // namespace cem
