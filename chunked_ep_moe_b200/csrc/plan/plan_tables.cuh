// Per-pass routing tables, built from the all-gathered [P, P, L] traffic matrix.
//
// The same __host__ __device__ code runs inside the single-CTA plan kernel and, for CPU tests,
// as a plain host function, so the table arithmetic is checked against the torch planner without
// a GPU. Semantics follow the reference planner (src/chunked_moe/plan.py:60-163): expert-major
// packed receive streams cut into S-row slices, max_r ceil(R_r / S) iterations on every rank.
//
// Everything is int32 and lives in ONE buffer (`PlanLayout` gives the offsets):
//
//   header[16]            [0] num_slices  [1] my stream rows  [2] max stream rows  [3] rows I send to remote ranks
//                         [4] 1 if num_slices exceeds max_slices  [5] my token copies T*K
//   send_start[P*L]       i = r*L+l : start of my rows for (receiver r, expert l) in my send order
//   seg_start[P*L]        i = r*L+l : where that segment starts in receiver r's stream
//   seg_size[P*L]         i = r*L+l : counts[me][r][l]
//   in_start[P*L]         i = s*L+l : where source s's segment for my expert l starts in MY stream
//   in_size[P*L]          i = s*L+l : counts[s][me][l]
//   src_send_start[P*L]   i = s*L+l : start of that segment in source s's send order (combine target)
//   expert_start[L], expert_rows[L]   my experts in my stream
//   per slice j:  num_mtiles[j], num_gtiles[j], num_chunks[j]
//                 mtiles[j][max_mtiles]  {expert, row0 (slice-relative), nrows, 0}         GEMM row tiles
//                 ptiles[j][max_ptiles]  {expert, row0, nrows (<= 256), 0}                 row-tile PAIRS (2-CTA GEMMs)
//                 gtiles[j][max_gtiles]  {expert, row0, nrows, flags}                      weight-grad groups
//                 put[j][P*L]            {send-order offset, rows, dest row, chunk prefix} my outgoing segments
#pragma once

#include <stdint.h>

#ifndef __CUDACC__
#define CEM_HD
#else
#define CEM_HD __host__ __device__
#endif

namespace cem {

constexpr int kPlanHeaderInts = 16;
constexpr int kTileM = 128;         // rows of one GEMM row tile
constexpr int kPutChunkRows = 4;    // rows one warp moves between two arrival signals

// gtile flags
constexpr int kGroupFirst = 1;  // the expert's rows begin in this slice: overwrite, do not accumulate
constexpr int kGroupFinal = 2;  // the expert's rows end in this slice: write the final gradient

struct PlanLayout {
  int P, L, S, max_slices, max_mtiles, max_gtiles, max_ptiles;
  int off_send_start, off_seg_start, off_seg_size, off_in_start, off_in_size, off_src_send_start;
  int off_expert_start, off_expert_rows;
  int off_num_mtiles, off_num_gtiles, off_num_chunks, off_num_ptiles;
  int off_mtiles, off_gtiles, off_put, off_ptiles;
  int total;
};

CEM_HD inline int plan_align4(int v) { return (v + 3) & ~3; }

CEM_HD inline PlanLayout make_plan_layout(int P, int L, int S, int max_slices) {
  PlanLayout y;
  y.P = P; y.L = L; y.S = S; y.max_slices = max_slices;
  y.max_mtiles = (S + kTileM - 1) / kTileM + L;
  y.max_gtiles = L;
  y.max_ptiles = (S + 2 * kTileM - 1) / (2 * kTileM) + L;
  const int n = P * L;
  int o = kPlanHeaderInts;
  y.off_send_start = o; o += plan_align4(n);
  y.off_seg_start = o; o += plan_align4(n);
  y.off_seg_size = o; o += plan_align4(n);
  y.off_in_start = o; o += plan_align4(n);
  y.off_in_size = o; o += plan_align4(n);
  y.off_src_send_start = o; o += plan_align4(n);
  y.off_expert_start = o; o += plan_align4(L);
  y.off_expert_rows = o; o += plan_align4(L);
  y.off_num_mtiles = o; o += plan_align4(max_slices);
  y.off_num_gtiles = o; o += plan_align4(max_slices);
  y.off_num_chunks = o; o += plan_align4(max_slices);
  y.off_num_ptiles = o; o += plan_align4(max_slices);
  y.off_mtiles = o; o += 4 * y.max_mtiles * max_slices;
  y.off_gtiles = o; o += 4 * y.max_gtiles * max_slices;
  y.off_put = o; o += 4 * n * max_slices;
  y.off_ptiles = o; o += 4 * y.max_ptiles * max_slices;
  y.total = o;
  return y;
}

CEM_HD inline int plan_clip(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// counts[s][r][l] -> count
CEM_HD inline int plan_count(const int* counts, int P, int L, int s, int r, int l) {
  return counts[(s * P + r) * L + l];
}

// Phase A: per-pass prefix sums. Threads stride over the P*L segment indices.
CEM_HD inline void plan_phase_a(const int* counts, int* plan, const PlanLayout& y, int me, int tid, int nthreads) {
  const int P = y.P, L = y.L, n = P * L;
  for (int i = tid; i < n; i += nthreads) {
    const int a = i / L, l = i % L;  // a is the receiver r (sender view) or the source s (receiver view)
    // --- sender view: segment (receiver a, expert l) -------------------------------------------
    int send_start = 0;
    for (int q = 0; q < i; ++q) send_start += counts[me * n + q];
    int seg_start = 0;  // recv_start[a][l][me]
    for (int lp = 0; lp < l; ++lp)
      for (int s = 0; s < P; ++s) seg_start += plan_count(counts, P, L, s, a, lp);
    for (int s = 0; s < me; ++s) seg_start += plan_count(counts, P, L, s, a, l);
    plan[y.off_send_start + i] = send_start;
    plan[y.off_seg_start + i] = seg_start;
    plan[y.off_seg_size + i] = plan_count(counts, P, L, me, a, l);
    // --- receiver view: segment (source a, my expert l) ----------------------------------------
    int in_start = 0;  // recv_start[me][l][a]
    for (int lp = 0; lp < l; ++lp)
      for (int s = 0; s < P; ++s) in_start += plan_count(counts, P, L, s, me, lp);
    for (int s = 0; s < a; ++s) in_start += plan_count(counts, P, L, s, me, l);
    int src_send_start = 0;  // send_start[a][me*L + l]
    for (int q = 0; q < me * L + l; ++q) src_send_start += counts[a * n + q];
    plan[y.off_in_start + i] = in_start;
    plan[y.off_in_size + i] = plan_count(counts, P, L, a, me, l);
    plan[y.off_src_send_start + i] = src_send_start;
  }
  for (int l = tid; l < L; l += nthreads) {
    int start = 0, rows = 0;
    for (int lp = 0; lp < l; ++lp)
      for (int s = 0; s < P; ++s) start += plan_count(counts, P, L, s, me, lp);
    for (int s = 0; s < P; ++s) rows += plan_count(counts, P, L, s, me, l);
    plan[y.off_expert_start + l] = start;
    plan[y.off_expert_rows + l] = rows;
  }
  if (tid == 0) {
    int max_rows = 0, my_rows = 0, remote = 0;
    for (int r = 0; r < P; ++r) {
      int rows = 0;
      for (int s = 0; s < P; ++s)
        for (int l = 0; l < L; ++l) rows += plan_count(counts, P, L, s, r, l);
      if (rows > max_rows) max_rows = rows;
      if (r == me) my_rows = rows;
      if (r != me)
        for (int l = 0; l < L; ++l) remote += plan_count(counts, P, L, me, r, l);
    }
    int num_slices = (max_rows + y.S - 1) / y.S;
    plan[0] = num_slices;
    plan[1] = my_rows;
    plan[2] = max_rows;
    plan[3] = remote;
    plan[4] = num_slices > y.max_slices ? 1 : 0;  // capacity overflow (the tables below are then truncated)
    int my_copies = 0;
    for (int q = 0; q < n; ++q) my_copies += counts[me * n + q];
    plan[5] = my_copies;  // T*K of this rank
    for (int q = 6; q < kPlanHeaderInts; ++q) plan[q] = 0;
  }
}

// Phase B: per-slice tables. Threads stride over slices. Needs phase A complete.
CEM_HD inline void plan_phase_b(int* plan, const PlanLayout& y, int tid, int nthreads) {
  const int P = y.P, L = y.L, S = y.S, n = P * L;
  int num_slices = plan[0];
  if (num_slices > y.max_slices) num_slices = y.max_slices;
  for (int j = tid; j < y.max_slices; j += nthreads) {
    int num_m = 0, num_g = 0, num_p = 0, chunks = 0;
    if (j < num_slices) {
      const int lo = j * S, hi = lo + S;
      int* mt = plan + y.off_mtiles + 4 * y.max_mtiles * j;
      int* gt = plan + y.off_gtiles + 4 * y.max_gtiles * j;
      int* pt = plan + y.off_ptiles + 4 * y.max_ptiles * j;
      for (int l = 0; l < L; ++l) {
        const int es = plan[y.off_expert_start + l], er = plan[y.off_expert_rows + l];
        const int first = plan_clip(lo, es, es + er), last = plan_clip(hi, es, es + er);
        const int rows = last - first;
        if (rows > 0) {
          for (int off = 0; off < rows; off += kTileM) {
            mt[4 * num_m + 0] = l;
            mt[4 * num_m + 1] = first - lo + off;
            mt[4 * num_m + 2] = rows - off < kTileM ? rows - off : kTileM;
            mt[4 * num_m + 3] = 0;
            ++num_m;
          }
          // Pairs of consecutive row tiles of one expert share its weights in a 2-CTA MMA; an odd
          // last tile is a pair whose second half is empty.
          for (int off = 0; off < rows; off += 2 * kTileM) {
            pt[4 * num_p + 0] = l;
            pt[4 * num_p + 1] = first - lo + off;
            pt[4 * num_p + 2] = rows - off < 2 * kTileM ? rows - off : 2 * kTileM;
            pt[4 * num_p + 3] = 0;
            ++num_p;
          }
          gt[4 * num_g + 0] = l;
          gt[4 * num_g + 1] = first - lo;
          gt[4 * num_g + 2] = rows;
          gt[4 * num_g + 3] = (es >= lo ? kGroupFirst : 0) | (es + er <= hi ? kGroupFinal : 0);
          ++num_g;
        } else if (j == 0 && er == 0) {
          // An expert nobody routed to still needs its gradient written (as zeros), exactly once.
          gt[4 * num_g + 0] = l;
          gt[4 * num_g + 1] = 0;
          gt[4 * num_g + 2] = 0;
          gt[4 * num_g + 3] = kGroupFirst | kGroupFinal;
          ++num_g;
        }
      }
      int* put = plan + y.off_put + 4 * n * j;
      for (int i = 0; i < n; ++i) {
        const int ss = plan[y.off_seg_start + i], sz = plan[y.off_seg_size + i];
        const int first = plan_clip(lo, ss, ss + sz), last = plan_clip(hi, ss, ss + sz);
        put[4 * i + 0] = plan[y.off_send_start + i] + (first - ss);
        put[4 * i + 1] = last - first;
        put[4 * i + 2] = first - lo;
        put[4 * i + 3] = chunks;
        chunks += (last - first + kPutChunkRows - 1) / kPutChunkRows;
      }
    }
    plan[y.off_num_mtiles + j] = num_m;
    plan[y.off_num_gtiles + j] = num_g;
    plan[y.off_num_chunks + j] = chunks;
    plan[y.off_num_ptiles + j] = num_p;
  }
}

}  // namespace cem
