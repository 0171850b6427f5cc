// Parameters of the grouped tcgen05 GEMM engine (one persistent kernel, six epilogues).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../common/status.cuh"
#include "../plan/plan_tables.cuh"

namespace cem {

// Tile shape of every mode: 128 x 256 accumulator (fp32 in TMEM, double buffered = all 512
// columns), K step 64 bf16 = one 128-byte swizzle span, 4-stage TMA pipeline.
constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kBlockK = 64;
constexpr int kStages = 4;
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;  // warp 0: TMA producer, warp 1: MMA issuer, warps 2-5: epilogue
constexpr int kRasterBand = 8;     // row tiles swept together across N so their A rows stay in L2

enum GemmMode : int {
  kModeSwiglu = 0,   // act = silu(x Wg) * (x Wu) from striped w_up; optional h          (replaces gmm_swiglu)
  kModeDownFwd = 1,  // y = act Wd; epilogue x router weight, rows stored to their source rank (gmm + combine)
  kModeDownDw = 2,   // backward remat of y: d_weight partials <g, y> and dy = w * g, y never stored
  kModeDswiglu = 3,  // d_act = dy Wd^T; epilogue SwiGLU' with h -> dh                     (gmm_dswiglu)
  kModeDx = 4,       // dx = dh Wu^T; rows (+ d_weight scalar) stored to their source rank  (gmm^T + combine)
  kModeTgmm = 5,     // dW[g] = lhs[rows_g]^T rhs[rows_g], fp32 carry across slices         (tgmm + accumulate)
};

// Per-CTA pipeline counters (SM cycles unless noted). They say which side of the operand ring waits for the other.
enum ProfSlot : int {
  kProfLoopCycles = 0,   // MMA warp: first tile started -> last MMA issued
  kProfLoopNs = 1,       // the same span in nanoseconds of the global timer (cycles / ns = SM clock in GHz)
  kProfEmptyWait = 2,    // producer: waiting for a free stage (the MMAs are the slower side)
  kProfFullWait = 3,     // MMA warp: waiting for a filled stage (the loads are the slower side)
  kProfAccWait = 4,      // MMA warp: waiting for the epilogue to hand an accumulator back
  kProfKBlocks = 5,      // k-blocks issued
  kProfEpiWait = 6,      // first epilogue warp: waiting for a finished accumulator
  kProfTiles = 7,        // tiles
  kProfSlots = 8,
};

struct GemmParams {
  // --- schedule ---------------------------------------------------------------------------
  const int* plan;   // per-pass plan buffer (see plan_tables.cuh)
  PlanLayout lay;
  int slice;         // slice index inside the pass
  int n_tiles;       // N / 256
  int m_tiles;       // tgmm: M / 128 (row tiles of the weight gradient); unused otherwise
  int k_blocks;      // gmm modes: K / 64
  int b_group_rows;  // rows one expert occupies in the flattened 2-D weight tensor map
  int me;            // this rank
  int stripe;        // SwiGLU stripe width (swiglu / dswiglu)
  uint32_t spin_limit;   // polls of a cross-GPU flag before giving up
  uint32_t mbar_limit;   // microseconds a pipeline barrier may take before giving up
  int suspend_waits;     // pair kernels: barriers completed from the partner CTA are waited for with try_wait, not polled
  int ret_blocked;       // combine modes: the return buffers are kept column tile by column tile (see run_epilogue)
  int ret_rows;          // rows of a return buffer (the stride between its column tiles in that layout)
  int ret_lsu;           // combine modes: staged rows leave with coalesced vector stores instead of bulk stores
  StatusBlock* status;
  // Optional pipeline counters of this mode, [grid][kProfSlots] summed over launches; null = not counted.
  unsigned long long* prof;
  // --- arrival flags (swiglu consumer) -----------------------------------------------------
  const uint32_t* arrive;     // [P*L] cumulative rows received per (source, local expert); null = no wait
  const uint32_t* pass_base;  // [P*L] value of `arrive` when this pass began
  // fp8 wire: rows are usable once the expansion kernel has released them, per local expert (replaces `arrive`)
  const uint32_t* ready;       // [L] cumulative rows expanded per local expert; null = not used
  const uint32_t* ready_base;  // [L] value of `ready` when this pass began
  // --- row-wise outputs / inputs (leading dims in elements) -----------------------------------
  __nv_bfloat16* out0;        // swiglu: act [S,F]; down_dw: dy [S,D]; dswiglu: dh [S,2F]
  __nv_bfloat16* out1;        // swiglu: h [S,2F] or null
  const __nv_bfloat16* in0;   // down_dw: g [S,D]; dswiglu: h [S,2F]
  const float* row_w;         // down_fwd / down_dw: router weight per slice row [S]
  float* dwp;                 // down_dw: out [S, n_tiles]; dx: in [S, dwp_tiles]
  int dwp_tiles;
  int ld0, ld1;
  // --- combine targets (down_fwd, dx) --------------------------------------------------------
  __nv_bfloat16* const* peer_rows;   // [P] base of each source rank's [T*K, ld] return buffer
  float* const* peer_dw;             // [P] base of each source rank's [T*K] d_weight rows (dx only)
  uint32_t* const* peer_count;       // [P] each source rank's returned-row counter
  // --- tgmm ---------------------------------------------------------------------------------
  const float* carry_in;   // [M, N] fp32 partial of the expert that straddles the previous slice boundary
  float* carry_out;        // [M, N] fp32 partial of the expert that straddles the next slice boundary
  __nv_bfloat16* grad_out; // [L, M, N] final gradient
};

// Dynamic shared memory the kernel asks for.
constexpr int kStageBytesA = kBlockM * kBlockK * 2;
constexpr int kStageBytesB = kBlockN * kBlockK * 2;
constexpr int kStageBytes = kStageBytesA + kStageBytesB;
// Epilogue staging, per epilogue warp: 16 rows x (512 bytes = the tile's 256 bf16 columns, + 16 bytes of padding so
// that the 16-byte pieces eight neighbouring lanes write at the same column fall into eight different bank groups);
// the weight-gradient mode uses the same space as two swizzled 4 KB blocks. The total leaves room for one small CTA
// of another kernel (a put, an fp8 expansion) beside a persistent GEMM CTA: 228 KB per SM, 1 KB reserved per CTA.
constexpr int kStageRowPitch = 528;
constexpr int kStagingBytes = 4 * 16 * kStageRowPitch;
static_assert(kStagingBytes >= 4 * 8192, "the weight-gradient mode stages two 4 KB blocks per epilogue warp");
constexpr int kSmemAlignSlack = 512;  // the kernels check at run time that the 1024-byte aligned layout fits
constexpr int kSmemTailBytes = 256;   // barriers, TMEM slot, flags
constexpr int kGemmSmemBytes = kSmemAlignSlack + kStages * kStageBytes + kStagingBytes + kSmemTailBytes;
static_assert(kGemmSmemBytes <= 232448, "more shared memory than one CTA can have");
static_assert(kGemmSmemBytes + 1024 + 1024 + 16 <= 233472, "no room for a second, small CTA on the SM");

// Extra dynamic shared memory (bytes) every GEMM launch asks for beyond what it uses. 0 leaves room for one small CTA
// of another kernel beside a persistent GEMM CTA; 1024 takes the SM's shared memory for the GEMM CTA alone (put and
// expansion kernels then only run on SMs a GEMM CTA has left). A measurement knob (`CEM_GEMM_EXCLUSIVE_SM=1`).
extern int g_gemm_extra_smem;
extern int g_pair_suspend_waits;  // CEM_PAIR_SUSPEND: see GemmParams::suspend_waits

// `map_c`: weight-gradient mode only, the bf16 gradient [L*M, N] with boxes of 32 rows x 64 columns (tiled stores);
// the other modes ignore it (pass any valid map).
void launch_grouped_gemm(int mode, const GemmParams& p, const CUtensorMap& map_a, const CUtensorMap& map_b,
                         const CUtensorMap& map_c, int grid, cudaStream_t stream);

// CTA-pair variant (clusters of two CTAs, one 256 x 256 MMA per pair). Same parameters; K-major weight
// maps must use 128-row boxes (each CTA loads its own half of the column tile). `grid` is rounded down
// to an even number.
extern int g_pair_grid_used;  // grid of the last CTA-pair launch (clamped to what is resident at once)
void launch_grouped_gemm_pair(int mode, const GemmParams& p, const CUtensorMap& map_a, const CUtensorMap& map_b,
                              const CUtensorMap& map_c, int grid, cudaStream_t stream);

}  // namespace cem
