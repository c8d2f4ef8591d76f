// C++ API of the single NVFP4 GEMM, source-compatible with the reference header
// include/sm120_nvfp4/gemm.hpp (names keep the _sm120 suffix although the kernels behind
// them are written for sm_100a / B200). Every function is a thin wrapper over the C ABI in
// b200_nvfp4.h; all pointers are device pointers owned by the caller, work is enqueued on
// `stream`, nothing is allocated and nothing synchronises.
#pragma once

#include <cstddef>
#include <cstdint>

#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

namespace sm120_nvfp4 {

// NVFP4 = packed E2M1 payload (two values per byte, low nibble first) with one UE4M3 scale
// per 16 consecutive K values; scale buffers use the 512-byte-atom block-scaled physical
// layout, not a flat [rows, K/16] array. The two element types are opaque one-byte tags
// (the reference aliases CUTLASS's float_e2m1_t / float_ue4m3_t here, gemm.hpp:16-17).
struct Nvfp4Element { std::uint8_t storage; };
struct Nvfp4Scale { std::uint8_t storage; };
using PackedStorage = std::uint8_t;
using OutputElement = half;

constexpr int kNvfp4ScaleVectorSize = 16;
constexpr int kScaleMNAlignment = 128;
constexpr int kInputAlignmentElements = 32;
constexpr int kOutputAlignmentElements = 8;

inline constexpr int ceil_div(int x, int y) { return (x + y - 1) / y; }
inline constexpr int align_up(int x, int alignment) { return ceil_div(x, alignment) * alignment; }

// Bytes of a packed row-major E2M1 matrix [rows, logical_cols].
inline constexpr std::size_t packed_fp4_bytes(int rows, int logical_cols) {
  return static_cast<std::size_t>(rows) * static_cast<std::size_t>(ceil_div(logical_cols, 2));
}

// Scale vectors along K, padded to a multiple of four (one atom holds four).
inline constexpr int scale_k_padded(int k) { return align_up(ceil_div(k, kNvfp4ScaleVectorSize), 4); }

// Bytes of one physical scale region of A ([m, k]) and of B ([n, k]).
inline constexpr std::size_t scale_a_elements(int m, int /*n*/, int k) {
  return static_cast<std::size_t>(align_up(m, kScaleMNAlignment)) * static_cast<std::size_t>(scale_k_padded(k));
}
inline constexpr std::size_t scale_b_elements(int /*m*/, int n, int k) {
  return static_cast<std::size_t>(align_up(n, kScaleMNAlignment)) * static_cast<std::size_t>(scale_k_padded(k));
}

enum class GemmStatus : int {
  kSuccess = 0,
  kInvalidArgument,
  kUnsupportedDevice,
  kInsufficientWorkspace,
  kCutlassNotSupported,
  kCutlassError,
  kCudaError,
};

const char* gemm_status_string(GemmStatus status);

enum class Nvfp4GemmPath : int {
  kGenericCute = 0,
  kM128SplitK4,
  kM256SplitK2,
};

const char* nvfp4_gemm_path_string(Nvfp4GemmPath path);

// Deterministic; does not look at the device.
Nvfp4GemmPath nvfp4_gemm_path_sm120(int m, int n, int k);

// Generic kernel, FP16 output: C[M,N] = (A * SFA) (B * SFB)^T.
GemmStatus nvfp4_cute_gemm_sm120(int m, int n, int k, const void* a, const void* b, const void* sfa,
                                 const void* sfb, half* c, cudaStream_t stream = nullptr);

// FP32 output: the FP32 accumulator is stored without narrowing.
GemmStatus nvfp4_cute_gemm_f32_sm120(int m, int n, int k, const void* a, const void* b,
                                     const void* sfa, const void* sfb, float* c,
                                     cudaStream_t stream = nullptr);

// Strided batch: operands [groups,M,K], [groups,N,K], outputs [groups,M,N]; one scale
// region per group.
GemmStatus nvfp4_cute_batched_gemm_sm120(int groups, int m, int n, int k, const void* a,
                                         const void* b, const void* sfa, const void* sfb, half* c,
                                         cudaStream_t stream = nullptr);

GemmStatus nvfp4_cute_batched_gemm_f32_sm120(int groups, int m, int n, int k, const void* a,
                                             const void* b, const void* sfa, const void* sfb,
                                             float* c, cudaStream_t stream = nullptr);

// The reference keeps a CUTLASS GemmUniversal instance behind these two names as a
// comparison path. This library ships no CUTLASS kernel: the workspace size is 0 and the
// call runs the same hand-written kernel as nvfp4_cute_gemm_sm120.
std::size_t nvfp4_cutlass_gemm_workspace_size_sm120(int m, int n, int k);

GemmStatus nvfp4_cutlass_gemm_sm120(int m, int n, int k, const void* a, const void* b,
                                    const void* sfa, const void* sfb, half* c, void* workspace,
                                    std::size_t workspace_bytes, cudaStream_t stream = nullptr);

// Workspace of the default path: split * M * N * 4 bytes for M == 128 (split 4) and
// M == 256 (split 2), else 0. Invalid shapes give 0 and are rejected at launch.
std::size_t nvfp4_gemm_workspace_size_sm120(int m, int n, int k);

// Default dispatcher: M == 128 / M == 256 take the split-K path, everything else the
// generic kernel. A is packed row-major [M,K], B packed row-major [N,K], C FP16 [M,N].
GemmStatus nvfp4_gemm_sm120(int m, int n, int k, const void* a, const void* b, const void* sfa,
                            const void* sfb, half* c, void* workspace, std::size_t workspace_bytes,
                            cudaStream_t stream = nullptr);

template <int N, int K>
inline GemmStatus nvfp4_gemm_sm120(int m, const void* a, const void* b, const void* sfa,
                                   const void* sfb, half* c, void* workspace,
                                   std::size_t workspace_bytes, cudaStream_t stream = nullptr) {
  return nvfp4_gemm_sm120(m, N, K, a, b, sfa, sfb, c, workspace, workspace_bytes, stream);
}

}  // namespace sm120_nvfp4
