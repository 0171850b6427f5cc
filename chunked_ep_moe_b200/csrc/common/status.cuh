// Device-side error reporting for bounded waits.
//
// No kernel in this library spins forever, traps or asserts. When a wait runs out (an mbarrier
// that never completes, an arrival flag nobody sets, a credit that never comes back) the kernel
// records what it was waiting for in a status block, unwinds and returns; the host reads the
// block after the pass and raises. The reference's semaphore waits are unbounded
// (src/chunked_moe/transport/nvshmem.py:144-177).
#pragma once

#include <stdint.h>

namespace cem {

enum StatusCode : int32_t {
  kStatusOk = 0,
  kStatusMbarTimeout = 1,     // an mbarrier phase never completed (TMA / MMA pipeline)
  kStatusArrivalTimeout = 2,  // dispatched rows never arrived (per-segment arrival counter)
  kStatusCreditTimeout = 3,   // a receiver never released its slice buffer
  kStatusReturnTimeout = 4,   // combined rows never came back
  kStatusBadIndex = 5,        // an index check failed; the access was skipped
  kStatusTrafficTimeout = 6,  // a peer's traffic-matrix row never arrived
};

enum KernelId : int32_t {
  kKernelGemm = 1,
  kKernelPut = 2,
  kKernelCombineReduce = 3,
  kKernelPlan = 4,
  kKernelWaitProbe = 5,
};

// 8 x int32, first writer wins (code != 0 means an error was recorded).
struct StatusBlock {
  int32_t code;
  int32_t kernel;
  int32_t mode;      // kernel-specific mode / role
  int32_t slice;     // slice sequence number or tile id
  int32_t detail;    // segment / peer / barrier index
  uint32_t expected;
  uint32_t seen;
  int32_t block;     // blockIdx.x of the reporter
};

#ifdef __CUDACC__
__device__ __forceinline__ void report_status(StatusBlock* st, int32_t code, int32_t kernel, int32_t mode,
                                              int32_t slice, int32_t detail, uint32_t expected, uint32_t seen) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0, code) == 0) {
    st->kernel = kernel;
    st->mode = mode;
    st->slice = slice;
    st->detail = detail;
    st->expected = expected;
    st->seen = seen;
    st->block = static_cast<int32_t>(blockIdx.x);
    __threadfence();
  }
}
#endif  // __CUDACC__

}  // namespace cem
