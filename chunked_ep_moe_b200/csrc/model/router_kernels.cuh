// Sigmoid top-k router (see router_kernels.cu). All tensors fp32 / int32, contiguous.
#pragma once

#include <cuda_runtime.h>

namespace cem {

// E a multiple of 32 up to 256, 1 <= top_k <= min(32, E).
bool router_supported(int E, int top_k);
// Grid of both kernels; `prob_partial` of the forward is [router_blocks(T), E].
int router_blocks(int T);
// logits [T, E], bias [E] -> ids [T, top_k] (descending score + bias, ties to the lower id), weights [T, top_k]
// (chosen sigmoid scores normalised over the chosen, times `scaling`), counts [E] += tokens per expert (integer
// atomics), prob_partial [blocks, E]: per block, the sum over its tokens of score / (sum of the token's scores).
void launch_router_fwd(const float* logits, const float* bias, int* ids, float* weights, int* counts,
                       float* prob_partial, int T, int E, int top_k, float scaling, cudaStream_t stream);
// d_weights [T, top_k], d_prob [E] (gradient w.r.t. the column sums of prob_partial) -> d_logits [T, E].
void launch_router_bwd(const float* logits, const int* ids, const float* d_weights, const float* d_prob,
                       float* d_logits, int T, int E, int top_k, float scaling, cudaStream_t stream);

}  // namespace cem
