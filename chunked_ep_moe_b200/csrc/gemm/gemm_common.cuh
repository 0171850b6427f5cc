// Pieces shared by the single-CTA and the CTA-pair GEMM kernels: tile decoding and the six fused epilogues.
#pragma once

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

// Dispatch consumer: waits until the rows of local expert `g` that belong to slices <= p.slice have arrived from every
// source rank (lane s watches source s), then orders the async proxy behind what was observed, because the rows were
// written through the generic proxy and TMA reads them next. Returns false on expiry (status recorded, abort set).
__device__ __forceinline__ bool wait_expert_rows(const GemmParams& p, int g, int lane, volatile int* abort_flag) {
  bool ok = true;
  if (p.ready != nullptr) {
    // fp8 wire: the expansion kernel releases an expert's rows (bf16, local) once they have arrived and been expanded.
    if (lane == 0) {
      const int through = plan_clip((p.slice + 1) * p.lay.S - p.plan[p.lay.off_expert_start + g], 0,
                                    p.plan[p.lay.off_expert_rows + g]);
      const uint32_t target = p.ready_base[g] + static_cast<uint32_t>(through);
      uint32_t seen = 0;
      ok = spin_until_reached(p.ready + g, target, p.spin_limit, &seen);
      if (!ok) {
        report_status(p.status, kStatusArrivalTimeout, kKernelGemm, kModeSwiglu, p.slice, 10000 + g, target, seen);
        *abort_flag = 1;
      }
    }
  } else if (lane < p.lay.P) {
    const int i = lane * p.lay.L + g;
    const int through = plan_clip((p.slice + 1) * p.lay.S - p.plan[p.lay.off_in_start + i], 0,
                                  p.plan[p.lay.off_in_size + i]);
    const uint32_t target = p.pass_base[i] + static_cast<uint32_t>(through);
    uint32_t seen = 0;
    ok = spin_until_reached(p.arrive + i, target, p.spin_limit, &seen);
    if (!ok) {
      report_status(p.status, kStatusArrivalTimeout, kKernelGemm, kModeSwiglu, p.slice, i, target, seen);
      *abort_flag = 1;
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  if (ok) fence_proxy_async_all();
  return ok;
}

// Sigmoid with the approximate divide (`__fdividef`: a reciprocal and a multiply, 2 ulp). The IEEE division the plain
// `/` compiles to is a subroutine of a dozen instructions, and in the SwiGLU epilogues it was most of the work per
// element; the results are rounded to bf16 right after, which has 16 bits less precision than the error made here.
__device__ __forceinline__ float sigmoid_f(float g) { return __fdividef(1.0f, 1.0f + __expf(-g)); }
__device__ __forceinline__ float silu_f(float g) { return g * sigmoid_f(g); }

// ---------------------------------------------------------------------------------------------
// Row blocks through the warp's staging buffer: 32 rows x 256 bytes, 16-byte pieces XOR-swizzled by row.
// The epilogues compute with one tile row per thread, but a warp access that touches 32 different rows costs the
// SM 32 requests towards L2, as many as 32 full lines; at 16-32 k-blocks per tile that request traffic, not the tensor
// pipe, set the pace. So row-wise inputs and outputs cross shared memory: threads read and write their own row in the
// staging block, and the warp moves the block to and from global memory 16 lanes per row (two full 256-byte row
// pieces per instruction, 8x fewer requests).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void stage_put(uint8_t* stage, int lane, int piece, int4 v) {
  *reinterpret_cast<int4*>(stage + lane * 256 + ((piece ^ (lane & 15)) << 4)) = v;
}

__device__ __forceinline__ int4 stage_get(const uint8_t* stage, int lane, int piece) {
  return *reinterpret_cast<const int4*>(stage + lane * 256 + ((piece ^ (lane & 15)) << 4));
}

// Staging block -> global: block row r goes to `gbase + r * ld_bytes` (256 bytes); rows >= nvalid are not stored.
// Shared-memory reads and global stores are issued as two batches: interleaved, every store would have to wait for the
// read before it and every read for the store before it (the compiler cannot tell that the two do not alias).
__device__ __forceinline__ void stage_flush(const uint8_t* stage, int lane, uint8_t* gbase, size_t ld_bytes,
                                            int nvalid) {
  __syncwarp();
  const int c16 = lane & 15, rhalf = lane >> 4;
#pragma unroll
  for (int batch = 0; batch < 2; ++batch) {
    int4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rsel = (batch * 8 + i) * 2 + rhalf;
      v[i] = *reinterpret_cast<const int4*>(stage + rsel * 256 + ((c16 ^ (rsel & 15)) << 4));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rsel = (batch * 8 + i) * 2 + rhalf;
      if (rsel < nvalid) *reinterpret_cast<int4*>(gbase + rsel * ld_bytes + c16 * 16) = v[i];
    }
  }
  __syncwarp();
}

// Global -> staging block in two steps, so that a caller can put work between the request and the use:
// `stage_fetch` issues all sixteen 16-byte loads of this lane at once (rows >= nvalid are not read and come out as zeros), `stage_commit` writes them to the staging block.
__device__ __forceinline__ void stage_fetch(int4 (&v)[16], int lane, const uint8_t* gbase, size_t ld_bytes,
                                            int nvalid) {
  const uint8_t* src = gbase + (lane >> 4) * ld_bytes + (lane & 15) * 16;
  const int mine = nvalid - (lane >> 4);  // this lane loads block rows rhalf, rhalf + 2, ...: those below nvalid
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    v[i] = make_int4(0, 0, 0, 0);
    if (2 * i < mine) v[i] = *reinterpret_cast<const int4*>(src + static_cast<size_t>(2 * i) * ld_bytes);
  }
}

__device__ __forceinline__ void stage_commit(uint8_t* stage, int lane, const int4 (&v)[16]) {
  __syncwarp();
  const int c16 = lane & 15, rhalf = lane >> 4;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int rsel = i * 2 + rhalf;
    *reinterpret_cast<int4*>(stage + rsel * 256 + ((c16 ^ (rsel & 15)) << 4)) = v[i];
  }
  __syncwarp();
}

// SwiGLU' goes through the staging block when a tile has fewer k-blocks than this (measured: 32 k-blocks per tile and
// below gain, 112 k-blocks per tile lose 3 % against the direct form with a one-chunk prefetch).
constexpr int kStagedDswigluMaxKBlocks = 64;

// Called by an epilogue warp BEFORE it waits for the tile's accumulator: asks L2 for the row-wise inputs the epilogue
// will read (the output gradient's columns for the down -> d_weight mode, the gate/up pre-activations for the
// SwiGLU' mode), so that the mainloop's duration hides their DRAM latency. Lane = tile row, as in the epilogue.
template <int MODE>
__device__ __forceinline__ void prefetch_epilogue_inputs(const GemmParams& p, const Tile& tl, int q, int lane) {
  if constexpr (MODE == kModeDownDw || MODE == kModeDswiglu) {
    const int row = q * 32 + lane;
    if (row >= tl.nrows) return;
    const size_t grow = static_cast<size_t>(tl.row0 + row);
    if constexpr (MODE == kModeDownDw) {
      const __nv_bfloat16* g_row = p.in0 + grow * p.ld0 + tl.n * kBlockN;  // 256 columns = four 128-byte lines
#pragma unroll
      for (int i = 0; i < 4; ++i) prefetch_l2(g_row + 64 * i);
    } else {
      const __nv_bfloat16* h_row = p.in0 + grow * p.ld0 + 2 * tl.n * kBlockN;  // the tile's 512 striped columns
#pragma unroll
      for (int i = 0; i < 8; ++i) prefetch_l2(h_row + 64 * i);
    }
  }
}

// `col0`, `ncols` (weight-gradient mode only): the accumulator columns this warp is responsible for; that mode may
// run two epilogue warps per TMEM lane quarter, each taking half of the columns.
// Epilogue of one 128 x 256 accumulator tile. `tacc` is this warp's TMEM address (lane quarter q, accumulator
// buffer), `tl` the tile as THIS CTA sees it (its 128 rows), `stage_gen` the warp's 8 KB staging buffer.
// `returned` (combine modes): lane s of every epilogue warp counts the row pieces this warp has stored to source
// rank s so far; `flush_returned` releases them once, after the CTA's last tile.
template <int MODE>
__device__ __forceinline__ void run_epilogue(const GemmParams& p, const Tile& tl, uint32_t tacc, int q, int lane,
                                             uint8_t* stage_gen, uint32_t& returned, const CUtensorMap* map_c,
                                             int col0 = 0, int ncols = kBlockN) {
  using Traits = ModeTraits<MODE>;
  const int row = q * 32 + lane;  // tile row owned by this thread
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
    // Two layouts of the return buffer. Row-major: a row's 512-byte piece of this tile goes to row `pos`, column tile
    // tl.n. Tile by tile ([column tile][row][256 columns], the 16-byte pieces of a row piece XOR-ed with pos & 7): the
    // pieces of CONSECUTIVE rows are then contiguous at the destination, and a run of rows of one source segment
    // leaves as one bulk store of up to 8 KB instead of one store per row (`combine_reduce` undoes the XOR).
    const bool blocked = p.ret_blocked != 0;
    if (src >= 0)
      dst = reinterpret_cast<unsigned long long>(
          blocked ? p.peer_rows[src] + (static_cast<size_t>(tl.n) * p.ret_rows + pos) * kBlockN
                  : p.peer_rows[src] + static_cast<size_t>(pos) * p.ld0 + tl.n * kBlockN);
    const bool lsu = p.ret_lsu != 0 && !blocked;
    const int sw = blocked ? (pos & 7) : (lsu ? (lane & 7) : 0);
    // Rows leave through the async proxy: a lane stages its WHOLE row of the tile (256 columns, 512 bytes) and hands it
    // to the copy engine as one bulk store to the source rank. The warp's staging holds 16 rows, so lanes 0-15 go first
    // and lanes 16-31 follow once the first sixteen stores have read their rows (TMEM is simply read twice). Nobody
    // waits for a remote store: the copy engine keeps the stores of consecutive tiles in flight while the warp goes
    // on to the next accumulator. Row pitch 528 bytes: eight neighbouring lanes hit eight different bank groups.
    uint8_t* my_row = stage_gen + (lane & 15) * ((blocked || lsu) ? 512 : kStageRowPitch);
    const uint32_t my_row_s = smem_u32(my_row);
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
      const bool mine = (lane >> 4) == pass;
      // The lane that used this staging row last (this lane or its partner 16 lanes away) has had it read.
      bulk_wait_read();
      __syncwarp();
#pragma unroll 1
      for (int c = 0; c < 8; c += 2) {
        uint32_t r2[32];
        tmem_ld_32x32(tacc + c * 32, r);
        tmem_ld_32x32(tacc + c * 32 + 32, r2);
        tmem_ld_wait();
        if (mine) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            *reinterpret_cast<int4*>(my_row + (((c * 4 + i) ^ sw) << 4)) =
                make_int4(pack_bf16(__uint_as_float(r[8 * i]) * w, __uint_as_float(r[8 * i + 1]) * w),
                          pack_bf16(__uint_as_float(r[8 * i + 2]) * w, __uint_as_float(r[8 * i + 3]) * w),
                          pack_bf16(__uint_as_float(r[8 * i + 4]) * w, __uint_as_float(r[8 * i + 5]) * w),
                          pack_bf16(__uint_as_float(r[8 * i + 6]) * w, __uint_as_float(r[8 * i + 7]) * w));
            *reinterpret_cast<int4*>(my_row + (((c * 4 + 4 + i) ^ sw) << 4)) =
                make_int4(pack_bf16(__uint_as_float(r2[8 * i]) * w, __uint_as_float(r2[8 * i + 1]) * w),
                          pack_bf16(__uint_as_float(r2[8 * i + 2]) * w, __uint_as_float(r2[8 * i + 3]) * w),
                          pack_bf16(__uint_as_float(r2[8 * i + 4]) * w, __uint_as_float(r2[8 * i + 5]) * w),
                          pack_bf16(__uint_as_float(r2[8 * i + 6]) * w, __uint_as_float(r2[8 * i + 7]) * w));
          }
        }
      }
      if (lsu) {
        // The warp writes the sixteen staged rows out itself, one whole 512-byte row per instruction (lane i moves
        // piece i): four full lines per store, nothing to wait for before the staging rows are reused.
        __syncwarp();
#pragma unroll 4
        for (int rr = 0; rr < 16; ++rr) {
          const unsigned long long d = __shfl_sync(0xffffffffu, dst, 16 * pass + rr);
          const int4 v = *reinterpret_cast<const int4*>(stage_gen + rr * 512 + ((lane ^ (rr & 7)) << 4));
          if (d != 0) *reinterpret_cast<int4*>(d + static_cast<unsigned long long>(lane) * 16) = v;
        }
        __syncwarp();
      } else if (!blocked) {
        if (mine) {
          fence_proxy_async_smem();
          if (dst != 0) bulk_store(dst, my_row_s, 512);
          bulk_commit();
        }
      } else {
        // Runs: consecutive lanes of this pass whose rows go to the same source at consecutive positions. The first
        // lane of a run stores the whole run (its rows are contiguous in the staging block and at the destination).
        if (mine) fence_proxy_async_smem();
        __syncwarp();
        const int prev_src = __shfl_up_sync(0xffffffffu, src, 1), prev_pos = __shfl_up_sync(0xffffffffu, pos, 1);
        const bool has = mine && dst != 0;
        const bool start = has && ((lane & 15) == 0 || prev_src != src || prev_pos + 1 != pos);
        const uint32_t breaks = __ballot_sync(0xffffffffu, mine && (start || dst == 0));
        if (start) {
          const uint32_t after = breaks & ~((2u << lane) - 1u);
          const int end = after ? (__ffs(after) - 1) : (16 * pass + 16);
          bulk_store(dst, my_row_s, static_cast<uint32_t>(end - lane) * 512u);
        }
        if (mine) bulk_commit();
      }
    }
    if constexpr (MODE == kModeDx) {
      if (tl.n == 0 && src >= 0) {
        float dw = 0.0f;
        for (int i = 0; i < p.dwp_tiles; ++i) dw += p.dwp[static_cast<size_t>(grow) * p.dwp_tiles + i];
        p.peer_dw[src][pos] = dw;
      }
    }
    // Lane s keeps the count of row pieces this warp has stored to source rank s; nothing is released here, so the
    // stores of consecutive tiles stay in flight together (`flush_returned` releases once, after the last tile).
    for (int s = 0; s < p.lay.P; ++s) {
      const uint32_t cnt = __popc(__ballot_sync(0xffffffffu, src == s));
      if (lane == s) returned += cnt;
    }
  } else if constexpr (MODE == kModeDownDw) {
    const float w = valid ? p.row_w[grow] : 0.0f;
    const int nvalid = plan_clip(tl.nrows - q * 32, 0, 32);
    const size_t block_off = static_cast<size_t>(tl.row0 + q * 32) * p.ld0 + tl.n * kBlockN;
    float partial = 0.0f;
    // Two 128-column halves: the warp brings its rows' g values into the staging block, every thread turns its own row
    // into dy = w * g in place (and adds its <g, y> share), the warp writes the block out as dy. The second half's g
    // values are requested before the first half is worked on.
    const uint8_t* g_block = reinterpret_cast<const uint8_t*>(p.in0 + block_off);
    int4 fetched[16];
    stage_fetch(fetched, lane, g_block, static_cast<size_t>(p.ld0) * 2, nvalid);
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      stage_commit(stage_gen, lane, fetched);
      if (half == 0) stage_fetch(fetched, lane, g_block + 256, static_cast<size_t>(p.ld0) * 2, nvalid);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        tmem_ld_32x32(tacc + half * 128 + c * 32, r);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int4 gv = stage_get(stage_gen, lane, c * 4 + i);
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
            stage_put(stage_gen, lane, c * 4 + i, make_int4(o[0], o[1], o[2], o[3]));
          }
        }
      }
      stage_flush(stage_gen, lane, reinterpret_cast<uint8_t*>(p.out0 + block_off + half * 128),
                  static_cast<size_t>(p.ld0) * 2, nvalid);
    }
    if (valid) p.dwp[static_cast<size_t>(grow) * p.dwp_tiles + tl.n] = partial;
  } else if constexpr (MODE == kModeDswiglu) {
    if (p.stripe <= 64 && p.k_blocks < kStagedDswigluMaxKBlocks) {
      // The tile's 512 striped columns of h / dh are four 128-column blocks; with stripes of 32 or 64 columns block b
      // holds the gate and up values of exactly the accumulator columns [64 b, 64 b + 64). The warp brings a block of h
      // into the staging buffer, every thread turns its own row into dh in place, the warp writes the block out.
      const int nvalid = plan_clip(tl.nrows - q * 32, 0, 32);
      const size_t block_off = static_cast<size_t>(tl.row0 + q * 32) * p.ld0 + 2 * tl.n * kBlockN;
      const int s8 = p.stripe >> 3;  // 16-byte pieces per stripe
      const uint8_t* h_block = reinterpret_cast<const uint8_t*>(p.in0 + block_off);
      const size_t ld_bytes = static_cast<size_t>(p.ld0) * 2;
      int4 fetched[16];
      stage_fetch(fetched, lane, h_block, ld_bytes, nvalid);
#pragma unroll 1
      for (int b = 0; b < 4; ++b) {
        stage_commit(stage_gen, lane, fetched);
        // The next block's h values are requested now and used after this block has been written out.
        if (b + 1 < 4) stage_fetch(fetched, lane, h_block + (b + 1) * 256, ld_bytes, nvalid);
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {  // 32 accumulator columns at a time
          tmem_ld_32x32(tacc + b * 64 + hh * 32, r);
          tmem_ld_wait();
          __syncwarp();
#pragma unroll
          for (int i4 = 0; i4 < 4; ++i4) {  // eight accumulator columns at a time
            if (!valid) break;
            const uint32_t* acc = r + 8 * i4;
            const int i = hh * 4 + i4;
            const int gpiece = (i / s8) * 2 * s8 + (i % s8), upiece = gpiece + s8;
            const int4 hg = stage_get(stage_gen, lane, gpiece), hu = stage_get(stage_gen, lane, upiece);
            const uint32_t gw[4] = {static_cast<uint32_t>(hg.x), static_cast<uint32_t>(hg.y),
                                    static_cast<uint32_t>(hg.z), static_cast<uint32_t>(hg.w)};
            const uint32_t uw[4] = {static_cast<uint32_t>(hu.x), static_cast<uint32_t>(hu.y),
                                    static_cast<uint32_t>(hu.z), static_cast<uint32_t>(hu.w)};
            uint32_t og[4], ou[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              // d_act is rounded to bf16 first, as the unfused reference stores it.
              const uint32_t db = pack_bf16(__uint_as_float(acc[2 * e]), __uint_as_float(acc[2 * e + 1]));
              float dg[2], du[2];
#pragma unroll
              for (int z = 0; z < 2; ++z) {
                const float d = z ? bf16_hi(db) : bf16_lo(db);
                const float gt = z ? bf16_hi(gw[e]) : bf16_lo(gw[e]);
                const float up = z ? bf16_hi(uw[e]) : bf16_lo(uw[e]);
                const float sig = sigmoid_f(gt);
                const float sl = gt * sig;
                dg[z] = d * up * (sig + sl * (1.0f - sig));
                du[z] = d * sl;
              }
              og[e] = pack_bf16(dg[0], dg[1]);
              ou[e] = pack_bf16(du[0], du[1]);
            }
            stage_put(stage_gen, lane, gpiece, make_int4(og[0], og[1], og[2], og[3]));
            stage_put(stage_gen, lane, upiece, make_int4(ou[0], ou[1], ou[2], ou[3]));
          }
        }
        stage_flush(stage_gen, lane, reinterpret_cast<uint8_t*>(p.out0 + block_off + b * 128),
                    static_cast<size_t>(p.ld0) * 2, nvalid);
      }
      return;
    }
    // Deep contractions (the epilogue hides behind the next tile either way and this form is a little cheaper), and
    // stripe 128 (a block of dh needs two blocks of h): the rows are read and written directly, one chunk ahead.
    const __nv_bfloat16* h_row = p.in0 + static_cast<size_t>(grow) * p.ld0;
    __nv_bfloat16* dh_row = p.out0 + static_cast<size_t>(grow) * p.ld0;
    auto gate_col = [&](int c) {  // striped column of the gate values that belong to accumulator chunk c
      const int f = tl.n * kBlockN + c * 32;
      const int b = f / p.stripe;
      return 2 * b * p.stripe + (f - b * p.stripe);
    };
    // The gate/up values of the NEXT 32 columns are requested before this chunk's accumulator is waited for, so their
    // global-load latency hides behind the TMEM load and the arithmetic (with 16-32 k-blocks per tile this epilogue,
    // not the mainloop, set the pace).
    int4 hg_next[4] = {}, hu_next[4] = {};
    if (valid) {
      const int g0 = gate_col(0);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        hg_next[i] = *reinterpret_cast<const int4*>(h_row + g0 + 8 * i);
        hu_next[i] = *reinterpret_cast<const int4*>(h_row + g0 + p.stripe + 8 * i);
      }
    }
#pragma unroll 1
    for (int c = 0; c < 8; ++c) {
      const int gcol = gate_col(c), ucol = gcol + p.stripe;
      int4 hg_cur[4], hu_cur[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { hg_cur[i] = hg_next[i]; hu_cur[i] = hu_next[i]; }
      tmem_ld_32x32(tacc + c * 32, r);
      if (valid && c + 1 < 8) {
        const int gn = gate_col(c + 1);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          hg_next[i] = *reinterpret_cast<const int4*>(h_row + gn + 8 * i);
          hu_next[i] = *reinterpret_cast<const int4*>(h_row + gn + p.stripe + 8 * i);
        }
      }
      tmem_ld_wait();
      if (valid) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int4 hg = hg_cur[i];
          const int4 hu = hu_cur[i];
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
              const float sig = sigmoid_f(gt);
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
    const size_t m_total = static_cast<size_t>(p.m_tiles) * kBlockM;
    const bool first = (tl.flags & kGroupFirst) != 0, final = (tl.flags & kGroupFinal) != 0;
    // The fp32 carry is private to this epilogue, so it is kept in the layout that suits it: tile by tile, and inside a
    // tile the 16-byte pieces (4 columns) of all 128 rows side by side. One warp load or store then covers 512
    // contiguous bytes (4 lines) instead of 32 rows 1 KB apart (32 requests at the SM's L2 port).
    const size_t tile_base = (static_cast<size_t>(tl.m) * p.n_tiles + tl.n) * (kBlockM * kBlockN);
    auto carry_off = [&](int col) { return tile_base + (static_cast<size_t>(col >> 2) * kBlockM + row) * 4; };
    auto load_chunk = [&](int col) {
      float4 pv[8];
      if (!first) {
#pragma unroll
        for (int i = 0; i < 8; ++i) pv[i] = *reinterpret_cast<const float4*>(p.carry_in + carry_off(col + 4 * i));
      }
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
          r[4 * i] = __float_as_uint(__uint_as_float(r[4 * i]) + pv[i].x);
          r[4 * i + 1] = __float_as_uint(__uint_as_float(r[4 * i + 1]) + pv[i].y);
          r[4 * i + 2] = __float_as_uint(__uint_as_float(r[4 * i + 2]) + pv[i].z);
          r[4 * i + 3] = __float_as_uint(__uint_as_float(r[4 * i + 3]) + pv[i].w);
        }
      }
    };
    if (final) {
      // bf16 gradient: the warp stages 32 rows x 64 columns at a time in the tensor map's swizzled layout (8 KB of
      // staging = two such blocks, so one block is filled while the other is being stored) and one lane hands each
      // block to the TMA as a tiled store: 16 stores of 4 KB per 128 x 256 tile, full lines, nobody waits for them.
      // (One 256-byte bulk store per lane and half tile was measured here and is slower: 256 small copies per tile
      // against ~4 k-blocks of MMA work.)
      const int out_row0 = tl.g * static_cast<int>(m_total) + tl.m * kBlockM + q * 32;  // in the [L*M, N] view
#pragma unroll 1
      for (int ch = 0; ch < ncols / 64; ++ch) {
        const int col = col0 + ch * 64;
        uint8_t* blk = stage_gen + (ch & 1) * 4096;
        if (lane == 0) bulk_wait_read_but_one();  // the store that last read this block is done with it
        __syncwarp();
        uint32_t r2[32];
        if (first && tl.kblocks > 0) {
          // Common case (the expert lies inside one slice): two TMEM loads per wait.
          tmem_ld_32x32(tacc + col, r);
          tmem_ld_32x32(tacc + col + 32, r2);
          tmem_ld_wait();
        } else {
          load_chunk(col + 32);
#pragma unroll
          for (int i = 0; i < 32; ++i) r2[i] = r[i];
          load_chunk(col);
        }
        uint8_t* my_row = blk + lane * 128;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          *reinterpret_cast<int4*>(my_row + ((i ^ (lane & 7)) << 4)) =
              make_int4(pack_bf16(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1])),
                        pack_bf16(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3])),
                        pack_bf16(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5])),
                        pack_bf16(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7])));
          *reinterpret_cast<int4*>(my_row + (((4 + i) ^ (lane & 7)) << 4)) =
              make_int4(pack_bf16(__uint_as_float(r2[8 * i]), __uint_as_float(r2[8 * i + 1])),
                        pack_bf16(__uint_as_float(r2[8 * i + 2]), __uint_as_float(r2[8 * i + 3])),
                        pack_bf16(__uint_as_float(r2[8 * i + 4]), __uint_as_float(r2[8 * i + 5])),
                        pack_bf16(__uint_as_float(r2[8 * i + 6]), __uint_as_float(r2[8 * i + 7])));
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(map_c, smem_u32(blk), tl.n * kBlockN + col, out_row0);
          bulk_commit();
        }
      }
    } else {
#pragma unroll 1
      for (int col = col0; col < col0 + ncols; col += 32) {
        load_chunk(col);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          *reinterpret_cast<float4*>(p.carry_out + carry_off(col + 4 * i)) =
              make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]),
                          __uint_as_float(r[4 * i + 3]));
      }
    }
  }
}

// Releases this warp's returned-row counts to their source ranks: every lane first waits until its own bulk stores
// have completed (the full wait, not the read-only one: the rows must have landed), the warp meets, and lane s then
// fences at system scope and adds its count to source s's counter.
__device__ __forceinline__ void flush_returned(const GemmParams& p, int lane, uint32_t returned) {
  bulk_wait_all();
  fence_proxy_async_all();
  __syncwarp();
  if (lane < p.lay.P && returned > 0) {
    __threadfence_system();
    red_add_release_sys(p.peer_count[lane], returned);
  }
}

}  // namespace
}  // namespace cem
