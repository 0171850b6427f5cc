// Expert sort for callers that must not allocate. This entry point has no counterpart in the
// reference (which sorts with XLA's argsort and lets XLA own every buffer).
//
// Who needs it: code that runs where cudaMalloc is off limits -- inside a region being captured
// into a CUDA graph, inside a memory-pool or allocator callback, in a process whose memory allowance
// is fixed up front by another framework, or in a latency-critical loop where an allocation
// (which may synchronise the device) is not acceptable. Such callers cannot hand the sort its
// scratch buffer either without allocating it somewhere, so the library carries the scratch
// itself: a fixed 1 MiB array in device memory that every GPU loading this library holds until
// the process exits.
//
// The call computes exactly what the library's regular expert sort computes:
//   order[p]        flat index (t*K + k) of the token copy at send-order position p
//                   (stable: copies of one expert keep ascending flat index)
//   inv_order[i]    send-order position of flat index i
//   counts[e]       number of copies routed to expert e
// from `expert_ids` (n int32 values in [0, num_experts)). All five pointers are device pointers
// on the current device; the caller owns inputs and outputs, the library owns only the scratch.
//
// Limits: 1 <= n <= 524288 ids, 1 <= num_experts <= 1024. Larger problems are rejected.
//
// Precondition: every id lies in [0, num_experts). The kernels never read or write out of bounds for other
// values, but such ids are left out of the sort: `counts` does not count them, their `inv_order` entries and
// the last entries of `order` keep whatever the buffers held before, and the call still returns 0. Validate
// ids before the call if they can be wrong.
//
// Return value: 0 on success; -1 null pointer; -2 n out of range; -3 num_experts out of range;
// any positive value is the cudaError_t of a failed runtime call (set-up or launch). The call does not clear
// the runtime's sticky error state: it reports an error that is pending when it returns, its own or an older
// one of the caller's, and leaves it pending.
//
// First call on a device: it looks up the device address of the scratch array (one runtime query,
// no allocation) and remembers it for that device. Make that first call outside of any stream
// capture; later calls only launch kernels on `stream`.
//
// Sharing: every call on a device uses the same scratch array and leaves its last contents in
// it. The kernels overwrite every scratch entry they read, so nothing needs clearing between
// calls -- but two calls that overlap on the GPU (different streams, no dependency) race on it.
// Order them on one stream or with events.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

int cem_expert_sort_noalloc(const int* expert_ids, int n, int num_experts, int* order, int* inv_order, int* counts,
                            cudaStream_t stream);

#ifdef __cplusplus
}
#endif
