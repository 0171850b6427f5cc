// Bandwidth-bound pieces of the decoder around the MoE layers, each as one kernel instead of a chain of framework
// elementwise kernels: residual add + RMSNorm (forward and backward), rotary embedding of q and k straight out of the
// fused qkv projection (forward and backward), and the cross-entropy of bf16 logits (forward and backward).
// The reference ships no model code (its host model lived in an external MaxText branch); these serve the trainer of
// `models/deepseek_tiny.py`.
#include "model_kernels.cuh"

#include <cuda_bf16.h>

namespace cem {

namespace {

__device__ __forceinline__ float bf_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t bf_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int kNormThreads = 256;  // 8 warps, one row per warp at a time
constexpr int kMaxNormUnits = 8;   // 16-byte units per lane: rows of up to 8 * 32 * 8 = 2048 columns

// s = x + delta (rounded to bf16, as the unfused residual add stores it); y = s * rsqrt(mean(s^2) + eps) * w.
__global__ void __launch_bounds__(kNormThreads) add_rms_norm_fwd_kernel(const __nv_bfloat16* x,
                                                                        const __nv_bfloat16* delta,
                                                                        const __nv_bfloat16* w, __nv_bfloat16* s_out,
                                                                        __nv_bfloat16* y, float* rstd_out, int rows,
                                                                        int cols, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int units = cols >> 3, per_lane = (units + 31) >> 5;
  for (int row = blockIdx.x * (kNormThreads / 32) + warp; row < rows; row += gridDim.x * (kNormThreads / 32)) {
    const int4* xr = reinterpret_cast<const int4*>(x + static_cast<size_t>(row) * cols);
    const int4* dr = delta ? reinterpret_cast<const int4*>(delta + static_cast<size_t>(row) * cols) : nullptr;
    float v[kMaxNormUnits][8];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < kMaxNormUnits; ++i) {
      const int u = lane + 32 * i;
      if (i < per_lane && u < units) {
        const int4 a = xr[u];
        const uint32_t aw[4] = {(uint32_t)a.x, (uint32_t)a.y, (uint32_t)a.z, (uint32_t)a.w};
        uint32_t bw[4] = {0, 0, 0, 0};
        if (dr) {
          const int4 b = dr[u];
          bw[0] = (uint32_t)b.x; bw[1] = (uint32_t)b.y; bw[2] = (uint32_t)b.z; bw[3] = (uint32_t)b.w;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float lo = bf_round(bf_lo(aw[e]) + bf_lo(bw[e])), hi = bf_round(bf_hi(aw[e]) + bf_hi(bw[e]));
          v[i][2 * e] = lo; v[i][2 * e + 1] = hi;
          ss += lo * lo + hi * hi;
        }
      }
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / cols + eps);
    if (lane == 0) rstd_out[row] = rstd;
    const int4* wr = reinterpret_cast<const int4*>(w);
    int4* sr = reinterpret_cast<int4*>(s_out + static_cast<size_t>(row) * cols);
    int4* yr = reinterpret_cast<int4*>(y + static_cast<size_t>(row) * cols);
#pragma unroll
    for (int i = 0; i < kMaxNormUnits; ++i) {
      const int u = lane + 32 * i;
      if (i < per_lane && u < units) {
        const int4 wv = wr[u];
        const uint32_t ww[4] = {(uint32_t)wv.x, (uint32_t)wv.y, (uint32_t)wv.z, (uint32_t)wv.w};
        uint32_t so[4], yo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          so[e] = bf_pack(v[i][2 * e], v[i][2 * e + 1]);
          yo[e] = bf_pack(v[i][2 * e] * rstd * bf_lo(ww[e]), v[i][2 * e + 1] * rstd * bf_hi(ww[e]));
        }
        if (delta) sr[u] = make_int4(so[0], so[1], so[2], so[3]);
        yr[u] = make_int4(yo[0], yo[1], yo[2], yo[3]);
      }
    }
  }
}

// ds = ds_in + rstd * (dy * w) - s * rstd^3 / D * sum(dy * w * s);  dw partial = sum over this block's rows of
// dy * s * rstd, one fp32 row per block (summed afterwards in fixed order).
__global__ void __launch_bounds__(kNormThreads) add_rms_norm_bwd_kernel(const __nv_bfloat16* dy,
                                                                        const __nv_bfloat16* ds_in,
                                                                        const __nv_bfloat16* s,
                                                                        const __nv_bfloat16* w, const float* rstd_in,
                                                                        __nv_bfloat16* ds_out, float* dw_partial,
                                                                        int rows, int cols) {
  extern __shared__ float s_dw[];  // [8 warps][cols]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int units = cols >> 3, per_lane = (units + 31) >> 5;
  float dw_acc[kMaxNormUnits][8];
#pragma unroll
  for (int i = 0; i < kMaxNormUnits; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) dw_acc[i][e] = 0.0f;
  const int4* wr = reinterpret_cast<const int4*>(w);
  for (int row = blockIdx.x * (kNormThreads / 32) + warp; row < rows; row += gridDim.x * (kNormThreads / 32)) {
    const int4* gr = reinterpret_cast<const int4*>(dy + static_cast<size_t>(row) * cols);
    const int4* sr = reinterpret_cast<const int4*>(s + static_cast<size_t>(row) * cols);
    const int4* ir = ds_in ? reinterpret_cast<const int4*>(ds_in + static_cast<size_t>(row) * cols) : nullptr;
    const float rstd = rstd_in[row];
    float gw[kMaxNormUnits][8], sv[kMaxNormUnits][8];
    float dot = 0.0f;
#pragma unroll
    for (int i = 0; i < kMaxNormUnits; ++i) {
      const int u = lane + 32 * i;
      if (i < per_lane && u < units) {
        const int4 g = gr[u], sx = sr[u], wv = wr[u];
        const uint32_t gq[4] = {(uint32_t)g.x, (uint32_t)g.y, (uint32_t)g.z, (uint32_t)g.w};
        const uint32_t sq[4] = {(uint32_t)sx.x, (uint32_t)sx.y, (uint32_t)sx.z, (uint32_t)sx.w};
        const uint32_t wq[4] = {(uint32_t)wv.x, (uint32_t)wv.y, (uint32_t)wv.z, (uint32_t)wv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float g0 = bf_lo(gq[e]), g1 = bf_hi(gq[e]), s0 = bf_lo(sq[e]), s1 = bf_hi(sq[e]);
          dw_acc[i][2 * e] += g0 * s0 * rstd;
          dw_acc[i][2 * e + 1] += g1 * s1 * rstd;
          gw[i][2 * e] = g0 * bf_lo(wq[e]); gw[i][2 * e + 1] = g1 * bf_hi(wq[e]);
          sv[i][2 * e] = s0; sv[i][2 * e + 1] = s1;
          dot += gw[i][2 * e] * s0 + gw[i][2 * e + 1] * s1;
        }
      }
    }
    dot = warp_sum(dot);
    const float coef = dot * rstd * rstd * rstd / cols;
    int4* outr = reinterpret_cast<int4*>(ds_out + static_cast<size_t>(row) * cols);
#pragma unroll
    for (int i = 0; i < kMaxNormUnits; ++i) {
      const int u = lane + 32 * i;
      if (i < per_lane && u < units) {
        uint32_t iq[4] = {0, 0, 0, 0};
        if (ir) {
          const int4 t = ir[u];
          iq[0] = (uint32_t)t.x; iq[1] = (uint32_t)t.y; iq[2] = (uint32_t)t.z; iq[3] = (uint32_t)t.w;
        }
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          o[e] = bf_pack(bf_lo(iq[e]) + gw[i][2 * e] * rstd - sv[i][2 * e] * coef,
                         bf_hi(iq[e]) + gw[i][2 * e + 1] * rstd - sv[i][2 * e + 1] * coef);
        outr[u] = make_int4(o[0], o[1], o[2], o[3]);
      }
    }
  }
  // Block-level sum of the eight warps' weight-gradient rows, then one row of partials per block.
#pragma unroll
  for (int i = 0; i < kMaxNormUnits; ++i) {
    const int u = lane + 32 * i;
    if (i < per_lane && u < units)
#pragma unroll
      for (int e = 0; e < 8; ++e) s_dw[warp * cols + u * 8 + e] = dw_acc[i][e];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float t = 0.0f;
#pragma unroll
    for (int wi = 0; wi < kNormThreads / 32; ++wi) t += s_dw[wi * cols + c];
    dw_partial[static_cast<size_t>(blockIdx.x) * cols + c] = t;
  }
}

// qkv [B, S, 3, H, hd] -> q, k (rotated) and v as contiguous [B, H, S, hd]. cos/sin: [S, hd/2] fp32.
// `inverse`: rotate by -theta and write back into the qkv layout (the backward).
template <bool kBackward>
__global__ void __launch_bounds__(256) rope_qkv_kernel(__nv_bfloat16* qkv, __nv_bfloat16* q, __nv_bfloat16* k,
                                                       __nv_bfloat16* v, const float* cos_t, const float* sin_t,
                                                       int B, int S, int H, int hd) {
  const int units = hd >> 3;  // 8 values = 4 rotation pairs per unit
  const size_t total = static_cast<size_t>(B) * S * H * units;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int u = static_cast<int>(idx % units);
    size_t rest = idx / units;
    const int h = static_cast<int>(rest % H); rest /= H;
    const int s = static_cast<int>(rest % S);
    const int b = static_cast<int>(rest / S);
    const size_t in_base = ((static_cast<size_t>(b) * S + s) * 3 * H + h) * hd + static_cast<size_t>(u) * 8;
    const size_t out_base = ((static_cast<size_t>(b) * H + h) * S + s) * hd + static_cast<size_t>(u) * 8;
    const float4 c = *reinterpret_cast<const float4*>(cos_t + static_cast<size_t>(s) * (hd >> 1) + u * 4);
    const float4 sn = *reinterpret_cast<const float4*>(sin_t + static_cast<size_t>(s) * (hd >> 1) + u * 4);
    const float cs[4] = {c.x, c.y, c.z, c.w};
    const float ss[4] = {kBackward ? -sn.x : sn.x, kBackward ? -sn.y : sn.y, kBackward ? -sn.z : sn.z,
                         kBackward ? -sn.w : sn.w};
#pragma unroll
    for (int part = 0; part < 2; ++part) {  // q then k
      __nv_bfloat16* rot = part == 0 ? q : k;
      const size_t in_off = in_base + static_cast<size_t>(part) * H * hd;
      const int4 raw = kBackward ? *reinterpret_cast<const int4*>(rot + out_base)
                                 : *reinterpret_cast<const int4*>(qkv + in_off);
      const uint32_t wds[4] = {(uint32_t)raw.x, (uint32_t)raw.y, (uint32_t)raw.z, (uint32_t)raw.w};
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float x1 = bf_lo(wds[e]), x2 = bf_hi(wds[e]);
        o[e] = bf_pack(x1 * cs[e] - x2 * ss[e], x1 * ss[e] + x2 * cs[e]);
      }
      const int4 res = make_int4(o[0], o[1], o[2], o[3]);
      if (kBackward) *reinterpret_cast<int4*>(qkv + in_off) = res;
      else *reinterpret_cast<int4*>(rot + out_base) = res;
    }
    const size_t v_off = in_base + static_cast<size_t>(2) * H * hd;
    if (kBackward) *reinterpret_cast<int4*>(qkv + v_off) = *reinterpret_cast<const int4*>(v + out_base);
    else *reinterpret_cast<int4*>(v + out_base) = *reinterpret_cast<const int4*>(qkv + v_off);
  }
}

// Cross-entropy of bf16 logits, one CTA per row: loss[row] = logsumexp(row) - row[target]; lse is kept for the backward.
__global__ void __launch_bounds__(256) cross_entropy_fwd_kernel(const __nv_bfloat16* logits, const int64_t* targets,
                                                                float* loss, float* lse_out, int cols) {
  __shared__ float s_m[8], s_s[8];
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int4* lr = reinterpret_cast<const int4*>(logits + static_cast<size_t>(row) * cols);
  const int units = cols >> 3;
  float m = -INFINITY, sum = 0.0f;  // online softmax: sum of exp(v - m)
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
    const int4 raw = lr[u];
    const uint32_t wds[4] = {(uint32_t)raw.x, (uint32_t)raw.y, (uint32_t)raw.z, (uint32_t)raw.w};
    float vals[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) { vals[2 * e] = bf_lo(wds[e]); vals[2 * e + 1] = bf_hi(wds[e]); }
    float mx = vals[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) mx = fmaxf(mx, vals[e]);
    const float nm = fmaxf(m, mx);
    float add = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) add += __expf(vals[e] - nm);
    sum = sum * __expf(m - nm) + add;
    m = nm;
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, sum, o);
    const float nm = fmaxf(m, om);
    sum = (nm == -INFINITY) ? 0.0f : sum * __expf(m - nm) + os * __expf(om - nm);
    m = nm;
  }
  if (lane == 0) { s_m[warp] = m; s_s[warp] = sum; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float fm = s_m[0], fs = s_s[0];
    for (int i = 1; i < 8; ++i) {
      const float nm = fmaxf(fm, s_m[i]);
      fs = (nm == -INFINITY) ? 0.0f : fs * __expf(fm - nm) + s_s[i] * __expf(s_m[i] - nm);
      fm = nm;
    }
    const float lse = fm + __logf(fs);
    lse_out[row] = lse;
    loss[row] = lse - __bfloat162float(logits[static_cast<size_t>(row) * cols + targets[row]]);
  }
}

// dlogits = (softmax - onehot(target)) * scale, bf16.
__global__ void __launch_bounds__(256) cross_entropy_bwd_kernel(const __nv_bfloat16* logits, const int64_t* targets,
                                                                const float* lse, const float* grad_scale,
                                                                __nv_bfloat16* dlogits, int cols) {
  const int row = blockIdx.x;
  const int4* lr = reinterpret_cast<const int4*>(logits + static_cast<size_t>(row) * cols);
  int4* dr = reinterpret_cast<int4*>(dlogits + static_cast<size_t>(row) * cols);
  const float l = lse[row], scale = *grad_scale;
  const int target = static_cast<int>(targets[row]);
  const int units = cols >> 3;
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
    const int4 raw = lr[u];
    const uint32_t wds[4] = {(uint32_t)raw.x, (uint32_t)raw.y, (uint32_t)raw.z, (uint32_t)raw.w};
    float p[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) { p[2 * e] = __expf(bf_lo(wds[e]) - l); p[2 * e + 1] = __expf(bf_hi(wds[e]) - l); }
    const int t = target - u * 8;
    if (t >= 0 && t < 8) p[t] -= 1.0f;
    dr[u] = make_int4(bf_pack(p[0] * scale, p[1] * scale), bf_pack(p[2] * scale, p[3] * scale),
                      bf_pack(p[4] * scale, p[5] * scale), bf_pack(p[6] * scale, p[7] * scale));
  }
}

// act = silu(gate) * up for gu = [gate | up] (two contiguous halves of `ffn` columns per row), eight columns a thread.
__global__ void __launch_bounds__(256) dense_swiglu_fwd_kernel(const __nv_bfloat16* gu, __nv_bfloat16* act,
                                                               size_t units, int ffn_units) {
  for (size_t u = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; u < units;
       u += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t row = u / ffn_units, c = u - row * ffn_units;
    const int4 g = reinterpret_cast<const int4*>(gu)[row * 2 * ffn_units + c];
    const int4 v = reinterpret_cast<const int4*>(gu)[row * 2 * ffn_units + ffn_units + c];
    const uint32_t gw[4] = {(uint32_t)g.x, (uint32_t)g.y, (uint32_t)g.z, (uint32_t)g.w};
    const uint32_t vw[4] = {(uint32_t)v.x, (uint32_t)v.y, (uint32_t)v.z, (uint32_t)v.w};
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float g0 = bf_lo(gw[e]), g1 = bf_hi(gw[e]);
      o[e] = bf_pack(g0 * __fdividef(1.0f, 1.0f + __expf(-g0)) * bf_lo(vw[e]),
                     g1 * __fdividef(1.0f, 1.0f + __expf(-g1)) * bf_hi(vw[e]));
    }
    reinterpret_cast<int4*>(act)[u] = make_int4(o[0], o[1], o[2], o[3]);
  }
}

// d_gu = [d_act * up * silu'(gate) | d_act * silu(gate)].
__global__ void __launch_bounds__(256) dense_swiglu_bwd_kernel(const __nv_bfloat16* gu, const __nv_bfloat16* d_act,
                                                               __nv_bfloat16* d_gu, size_t units, int ffn_units) {
  for (size_t u = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; u < units;
       u += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t row = u / ffn_units, c = u - row * ffn_units;
    const size_t gi = row * 2 * ffn_units + c, vi = gi + ffn_units;
    const int4 g = reinterpret_cast<const int4*>(gu)[gi];
    const int4 v = reinterpret_cast<const int4*>(gu)[vi];
    const int4 d = reinterpret_cast<const int4*>(d_act)[u];
    const uint32_t gw[4] = {(uint32_t)g.x, (uint32_t)g.y, (uint32_t)g.z, (uint32_t)g.w};
    const uint32_t vw[4] = {(uint32_t)v.x, (uint32_t)v.y, (uint32_t)v.z, (uint32_t)v.w};
    const uint32_t dw[4] = {(uint32_t)d.x, (uint32_t)d.y, (uint32_t)d.z, (uint32_t)d.w};
    uint32_t og[4], ov[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float dg[2], dv[2];
#pragma unroll
      for (int z = 0; z < 2; ++z) {
        const float gt = z ? bf_hi(gw[e]) : bf_lo(gw[e]);
        const float up = z ? bf_hi(vw[e]) : bf_lo(vw[e]);
        const float da = z ? bf_hi(dw[e]) : bf_lo(dw[e]);
        const float sig = __fdividef(1.0f, 1.0f + __expf(-gt));
        const float sl = gt * sig;
        dg[z] = da * up * (sig + sl * (1.0f - sig));
        dv[z] = da * sl;
      }
      og[e] = bf_pack(dg[0], dg[1]);
      ov[e] = bf_pack(dv[0], dv[1]);
    }
    reinterpret_cast<int4*>(d_gu)[gi] = make_int4(og[0], og[1], og[2], og[3]);
    reinterpret_cast<int4*>(d_gu)[vi] = make_int4(ov[0], ov[1], ov[2], ov[3]);
  }
}

}  // namespace

void launch_add_rms_norm_fwd(const void* x, const void* delta, const void* w, void* s_out, void* y, float* rstd,
                             int rows, int cols, float eps, cudaStream_t stream) {
  int grid = (rows + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  if (grid < 1) grid = 1;
  add_rms_norm_fwd_kernel<<<grid, kNormThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(delta),
      static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(s_out), static_cast<__nv_bfloat16*>(y), rstd,
      rows, cols, eps);
}

int add_rms_norm_bwd_blocks(int rows) {
  int grid = (rows + 7) / 8;
  if (grid > 148 * 2) grid = 148 * 2;
  return grid < 1 ? 1 : grid;
}

void launch_add_rms_norm_bwd(const void* dy, const void* ds_in, const void* s, const void* w, const float* rstd,
                             void* ds_out, float* dw_partial, int rows, int cols, cudaStream_t stream) {
  const int grid = add_rms_norm_bwd_blocks(rows);
  const size_t smem = static_cast<size_t>(kNormThreads / 32) * cols * sizeof(float);
  static bool configured = false;
  if (!configured) {  // 64 KB at 2048 columns: above the default limit
    cudaFuncSetAttribute(add_rms_norm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
    configured = true;
  }
  add_rms_norm_bwd_kernel<<<grid, kNormThreads, smem, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(ds_in),
      static_cast<const __nv_bfloat16*>(s), static_cast<const __nv_bfloat16*>(w), rstd,
      static_cast<__nv_bfloat16*>(ds_out), dw_partial, rows, cols);
}

void launch_rope_qkv(void* qkv, void* q, void* k, void* v, const float* cos_t, const float* sin_t, int B, int S, int H,
                     int hd, bool backward, cudaStream_t stream) {
  const size_t total = static_cast<size_t>(B) * S * H * (hd >> 3);
  int grid = static_cast<int>((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  if (grid < 1) grid = 1;
  if (backward)
    rope_qkv_kernel<true><<<grid, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(qkv), static_cast<__nv_bfloat16*>(q),
                                                    static_cast<__nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(v),
                                                    cos_t, sin_t, B, S, H, hd);
  else
    rope_qkv_kernel<false><<<grid, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(qkv), static_cast<__nv_bfloat16*>(q),
                                                     static_cast<__nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(v),
                                                     cos_t, sin_t, B, S, H, hd);
}

void launch_cross_entropy_fwd(const void* logits, const int64_t* targets, float* loss, float* lse, int rows, int cols,
                              cudaStream_t stream) {
  cross_entropy_fwd_kernel<<<rows, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), targets, loss, lse,
                                                     cols);
}

void launch_cross_entropy_bwd(const void* logits, const int64_t* targets, const float* lse, const float* grad_scale,
                              void* dlogits, int rows, int cols, cudaStream_t stream) {
  cross_entropy_bwd_kernel<<<rows, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), targets, lse,
                                                     grad_scale, static_cast<__nv_bfloat16*>(dlogits), cols);
}

void launch_dense_swiglu(const void* gu, const void* d_act, void* out, int rows, int ffn, bool backward,
                         cudaStream_t stream) {
  const size_t units = static_cast<size_t>(rows) * (ffn >> 3);
  if (units == 0) return;
  int grid = static_cast<int>((units + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  if (backward)
    dense_swiglu_bwd_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(gu),
                                                      static_cast<const __nv_bfloat16*>(d_act),
                                                      static_cast<__nv_bfloat16*>(out), units, ffn >> 3);
  else
    dense_swiglu_fwd_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(gu),
                                                      static_cast<__nv_bfloat16*>(out), units, ffn >> 3);
}

}  // namespace cem
