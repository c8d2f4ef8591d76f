// Split-K NVFP4 GEMM whose partial-sum scratch lives inside the library.
//
// b200_nvfp4_gemm_splitk wants a caller-provided FP32 workspace of split_k * M * N floats. Some
// callers have no way to provide one at the point of the call: a plugin hook that is handed
// only its operand pointers and a stream, a host runtime with a frozen memory plan, or a
// process that must not touch the device allocator on its serving path because an allocation
// can synchronise the whole device. For them this file keeps one fixed scratch array in the
// module's device data segment and runs the same two kernels (split-K GEMM slices, then the
// ordered reduction) on it. Nothing here, or below it, allocates device or host-pinned memory.
//
// Limits and rules of use:
//   * split_k * M * N <= kScratchFloats (4 Mi floats = 16 MiB); larger problems are refused with
//     B200_NVFP4_INSUFFICIENT_WORKSPACE and must use the workspace-taking entry point.
//   * The array exists once per device. Two calls that overlap in time on one device (different
//     streams or host threads) write the same scratch and race; serialise them on one stream or
//     with events. Calls on different devices do not interact.
//   * The first call on each device looks the array's address up (a host-side query, no launch)
//     and caches it; make that first call before any stream capture is started.
//   * Nothing in the scratch has to be cleared: every call writes each partial sum it later
//     reads (a k-split without work writes zeros), so stale contents never reach the output.
#include <cstddef>
#include <cstdint>
#include <mutex>

#include <cuda_runtime.h>

#include "b200_nvfp4.h"
#include "internal.hpp"

namespace b200 {
namespace {

constexpr size_t kScratchFloats = size_t{4} << 20;

static __device__ __align__(256) float g_splitk_scratch[kScratchFloats];

// Address of g_splitk_scratch on the current device, looked up once per device with that
// device current. Returns nullptr (and the CUDA error stays readable by the caller through the
// status code) when the lookup fails.
float* splitk_scratch_for_current_device() {
  constexpr int kMaxDevices = 64;
  static float* cache[kMaxDevices] = {};
  static std::mutex mu;
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (cache[device] == nullptr) {
    float* ptr = nullptr;
    if (cudaGetSymbolAddress((void**)&ptr, g_splitk_scratch) != cudaSuccess) return nullptr;
    cache[device] = ptr;
  }
  return cache[device];
}

}  // namespace
}  // namespace b200

extern "C" {

size_t b200_nvfp4_gemm_splitk_static_max_elements(void) { return b200::kScratchFloats; }

int b200_nvfp4_gemm_splitk_static(int m, int n, int k, int split_k, const void* a, const void* b,
                                  const void* sfa, const void* sfb, void* c_f16,
                                  b200_stream_t stream) {
  // split_k is bounded first (a 128-wide k-tile per split at least), so that the element count
  // below is a product of bounded factors; each multiplication is checked against the limit by
  // division before it is made (cf. the reference's workspace arithmetic,
  // src/gemm/specialized/m128_gemm.cu:403-414), so huge M or N cannot wrap around into range.
  if (m <= 0 || n <= 0 || k <= 0 || split_k < 1 || split_k > (k + 127) / 128) return B200_NVFP4_INVALID_ARGUMENT;
  const size_t per_row = b200::kScratchFloats / static_cast<size_t>(n);        // floats of scratch per output row
  if (per_row == 0 || static_cast<size_t>(m) > per_row) return B200_NVFP4_INSUFFICIENT_WORKSPACE;
  const size_t slice = static_cast<size_t>(m) * static_cast<size_t>(n);        // <= kScratchFloats
  if (static_cast<size_t>(split_k) > b200::kScratchFloats / slice) return B200_NVFP4_INSUFFICIENT_WORKSPACE;
  float* scratch = b200::splitk_scratch_for_current_device();
  if (scratch == nullptr) return B200_NVFP4_CUDA_ERROR;
  return b200::gemm_splitk(m, n, k, split_k, a, b, sfa, sfb, c_f16, scratch,
                           b200::kScratchFloats * sizeof(float), static_cast<cudaStream_t>(stream));
}

}  // extern "C"
