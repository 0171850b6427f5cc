// Allocation-free expert sort: the library's sort kernels run on a scratch array that lives in
// this file's device data segment instead of a buffer somebody had to allocate.
#include "expert_sort_noalloc.h"

#include <mutex>

#include "plan_kernel.cuh"

namespace {

constexpr int kMaxIds = 524288;     // 256 sort blocks of 2048 ids
constexpr int kMaxExperts = 1024;
constexpr int kMaxBlocks = kMaxIds / 2048;
constexpr int kMaxDevices = 64;

// Per-(expert, block) histogram / offset table of the counting sort: 256 x 1024 int32 = 1 MiB.
// In host code this name is only a handle for the runtime, never a device address.
static __device__ __align__(256) int g_sort_scratch[kMaxBlocks * kMaxExperts];

std::mutex g_mutex;
int* g_scratch_on_device[kMaxDevices] = {};

// Device address of the scratch array on the current device (queried once per device).
cudaError_t scratch_address(int** out) {
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_scratch_on_device[dev] == nullptr) {
    int* ptr = nullptr;
    err = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_sort_scratch);
    if (err != cudaSuccess) return err;
    g_scratch_on_device[dev] = ptr;
  }
  *out = g_scratch_on_device[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" int cem_expert_sort_noalloc(const int* expert_ids, int n, int num_experts, int* order, int* inv_order,
                                       int* counts, cudaStream_t stream) {
  if (expert_ids == nullptr || order == nullptr || inv_order == nullptr || counts == nullptr) return -1;
  if (n < 1 || n > kMaxIds) return -2;
  if (num_experts < 1 || num_experts > kMaxExperts) return -3;
  if (cem::expert_sort_scratch_ints(n, num_experts) > static_cast<size_t>(kMaxBlocks) * kMaxExperts) return -2;
  int* scratch = nullptr;
  cudaError_t err = scratch_address(&scratch);
  if (err != cudaSuccess) return static_cast<int>(err);
  // Every (expert, block) entry the scan and scatter kernels read is first written by the histogram
  // kernel of this same call, so stale contents from an earlier call are never observed.
  cem::launch_expert_sort(expert_ids, n, num_experts, order, inv_order, counts, scratch, stream);
  // Peek, not get: an error some earlier call of the caller left behind stays where it is.
  err = cudaPeekAtLastError();
  return err == cudaSuccess ? 0 : static_cast<int>(err);
}
