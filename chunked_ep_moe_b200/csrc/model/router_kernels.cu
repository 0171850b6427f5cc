// Sigmoid top-k router as two kernels (forward, backward), one warp per token.
//
// What the decoder's router does after its logits GEMM (sigmoid scores, selection by score + bias, the chosen scores
// normalised and scaled, per-expert load counts and the mean normalised score per expert for the balance loss) is a
// dozen framework kernels forward and two dozen backward on [T, E] tensors of a few MB; here a warp keeps a token's E
// scores in registers (E / 32 per lane) and does all of it in one pass. Everything is deterministic: the top-k breaks
// ties towards the lower expert id, load counts are integer atomics, and the per-expert score sums are reduced in a
// fixed order (per warp over its rows, per block over its warps, then over blocks by the caller).
#include "router_kernels.cuh"

#include <math_constants.h>

namespace cem {

namespace {

constexpr int kRouterWarps = 8;
constexpr int kRouterMaxPerLane = 8;  // E <= 256

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

template <int V>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_fwd_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int* __restrict__ ids,
                  float* __restrict__ weights, int* __restrict__ counts, float* __restrict__ prob_partial, int T,
                  int top_k, float scaling) {
  constexpr int E = V * 32;
  __shared__ float s_acc[kRouterWarps][E];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gw = blockIdx.x * kRouterWarps + warp, nw = gridDim.x * kRouterWarps;
  float b[V], acc[V];
#pragma unroll
  for (int v = 0; v < V; ++v) {
    b[v] = bias[v * 32 + lane];
    acc[v] = 0.0f;
  }
  for (int t = gw; t < T; t += nw) {
    float s[V], key[V];
    float row = 0.0f;
#pragma unroll
    for (int v = 0; v < V; ++v) {
      s[v] = 1.0f / (1.0f + __expf(-logits[static_cast<size_t>(t) * E + v * 32 + lane]));
      key[v] = s[v] + b[v];
      row += s[v];
    }
    row = fmaxf(warp_sum_f(row), 1e-20f);
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] += s[v] / row;
    int my_id = 0;
    float my_score = 0.0f, chosen_sum = 0.0f;
    for (int k = 0; k < top_k; ++k) {
      float best = -CUDART_INF_F;
      int best_e = E;
#pragma unroll
      for (int v = 0; v < V; ++v) {
        if (key[v] > best) {  // ascending v = ascending expert id: the first maximum wins inside a lane
          best = key[v];
          best_e = v * 32 + lane;
        }
      }
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, d);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, d);
        if (ob > best || (ob == best && oe < best_e)) {
          best = ob;
          best_e = oe;
        }
      }
      float sc = 0.0f;
#pragma unroll
      for (int v = 0; v < V; ++v) {
        if (best_e == v * 32 + lane) {
          sc = s[v];
          key[v] = -CUDART_INF_F;
        }
      }
      sc = __shfl_sync(0xffffffffu, sc, best_e & 31);
      chosen_sum += sc;
      if (lane == k) {
        my_id = best_e;
        my_score = sc;
      }
    }
    if (lane < top_k) {
      ids[static_cast<size_t>(t) * top_k + lane] = my_id;
      weights[static_cast<size_t>(t) * top_k + lane] = my_score / fmaxf(chosen_sum, 1e-20f) * scaling;
      atomicAdd(counts + my_id, 1);
    }
  }
#pragma unroll
  for (int v = 0; v < V; ++v) s_acc[warp][v * 32 + lane] = acc[v];
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float sum = 0.0f;
#pragma unroll
    for (int w = 0; w < kRouterWarps; ++w) sum += s_acc[w][e];
    prob_partial[static_cast<size_t>(blockIdx.x) * E + e] = sum;
  }
}

template <int V>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_bwd_kernel(const float* __restrict__ logits, const int* __restrict__ ids, const float* __restrict__ d_weights,
                  const float* __restrict__ d_prob, float* __restrict__ d_logits, int T, int top_k, float scaling) {
  constexpr int E = V * 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gw = blockIdx.x * kRouterWarps + warp, nw = gridDim.x * kRouterWarps;
  float gp[V];
#pragma unroll
  for (int v = 0; v < V; ++v) gp[v] = d_prob[v * 32 + lane];
  for (int t = gw; t < T; t += nw) {
    float s[V], ds[V];
    float row = 0.0f, gdot = 0.0f;
#pragma unroll
    for (int v = 0; v < V; ++v) {
      s[v] = 1.0f / (1.0f + __expf(-logits[static_cast<size_t>(t) * E + v * 32 + lane]));
      row += s[v];
      gdot += gp[v] * s[v];
    }
    row = warp_sum_f(row);
    gdot = warp_sum_f(gdot);
    // prob_e = sum_t s_te / max(row_t, tiny): below the clamp the denominator is a constant.
    const bool clamped = row < 1e-20f;
    const float inv = 1.0f / fmaxf(row, 1e-20f);
#pragma unroll
    for (int v = 0; v < V; ++v) ds[v] = gp[v] * inv - (clamped ? 0.0f : gdot * inv * inv);
    // weights_k = scaling * s_k / max(sum of the chosen, tiny)
    int my_id = -1;
    float my_dw = 0.0f;
    if (lane < top_k) {
      my_id = ids[static_cast<size_t>(t) * top_k + lane];
      my_dw = d_weights[static_cast<size_t>(t) * top_k + lane];
    }
    float chosen = 0.0f, wdot = 0.0f;
    for (int k = 0; k < top_k; ++k) {
      const int e = __shfl_sync(0xffffffffu, my_id, k);
      const float dw = __shfl_sync(0xffffffffu, my_dw, k);
      float sc = 0.0f;
#pragma unroll
      for (int v = 0; v < V; ++v)
        if (e == v * 32 + lane) sc = s[v];
      sc = __shfl_sync(0xffffffffu, sc, e & 31);
      chosen += sc;
      wdot += dw * sc;
    }
    const bool clamped_sel = chosen < 1e-20f;
    const float inv_sel = 1.0f / fmaxf(chosen, 1e-20f);
    for (int k = 0; k < top_k; ++k) {
      const int e = __shfl_sync(0xffffffffu, my_id, k);
      const float dw = __shfl_sync(0xffffffffu, my_dw, k);
      const float g = scaling * (dw * inv_sel - (clamped_sel ? 0.0f : wdot * inv_sel * inv_sel));
#pragma unroll
      for (int v = 0; v < V; ++v)
        if (e == v * 32 + lane) ds[v] += g;
    }
#pragma unroll
    for (int v = 0; v < V; ++v)
      d_logits[static_cast<size_t>(t) * E + v * 32 + lane] = ds[v] * s[v] * (1.0f - s[v]);
  }
}

}  // namespace

int router_blocks(int T) {
  const int want = (T + kRouterWarps - 1) / kRouterWarps;
  return want < 1 ? 1 : (want > 296 ? 296 : want);
}

bool router_supported(int E, int top_k) {
  return E >= 32 && E % 32 == 0 && E / 32 <= kRouterMaxPerLane && top_k >= 1 && top_k <= 32 && top_k <= E;
}

#define CEM_ROUTER_DISPATCH(V, CALL) \
  switch (V) {                       \
    case 1: { constexpr int kV = 1; CALL; break; } \
    case 2: { constexpr int kV = 2; CALL; break; } \
    case 3: { constexpr int kV = 3; CALL; break; } \
    case 4: { constexpr int kV = 4; CALL; break; } \
    case 5: { constexpr int kV = 5; CALL; break; } \
    case 6: { constexpr int kV = 6; CALL; break; } \
    case 7: { constexpr int kV = 7; CALL; break; } \
    case 8: { constexpr int kV = 8; CALL; break; } \
    default: break;                  \
  }

void launch_router_fwd(const float* logits, const float* bias, int* ids, float* weights, int* counts,
                       float* prob_partial, int T, int E, int top_k, float scaling, cudaStream_t stream) {
  const int blocks = router_blocks(T);
  CEM_ROUTER_DISPATCH(E / 32, (router_fwd_kernel<kV><<<blocks, kRouterWarps * 32, 0, stream>>>(
                                  logits, bias, ids, weights, counts, prob_partial, T, top_k, scaling)));
}

void launch_router_bwd(const float* logits, const int* ids, const float* d_weights, const float* d_prob,
                       float* d_logits, int T, int E, int top_k, float scaling, cudaStream_t stream) {
  const int blocks = router_blocks(T);
  CEM_ROUTER_DISPATCH(E / 32, (router_bwd_kernel<kV><<<blocks, kRouterWarps * 32, 0, stream>>>(
                                  logits, ids, d_weights, d_prob, d_logits, T, top_k, scaling)));
}

}  // namespace cem
