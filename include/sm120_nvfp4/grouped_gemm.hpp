// C++ API of the expert-grouped NVFP4 GEMM, source-compatible with the reference header
// include/sm120_nvfp4/grouped_gemm.hpp:15-21.
#pragma once

#include <cuda_runtime_api.h>

namespace sm120_nvfp4 {
namespace grouped_gemm {

// y[cu_seqlens[e] + r, :] = x_e[r, :] * w[e]^T for r < seqlens[e], FP16.
// x / w hold two E2M1 values per byte; x_scale has one region of m_scale_pad rows per group
// (indexed by the row inside the group), w_scale one region of align128(n) rows per group.
// tmas_ptr, tiles_ptr and cu_tiles_ptr are the per-call scratch of the reference ABI:
// tmas_ptr is not used by this implementation, tiles_ptr / cu_tiles_ptr receive the
// per-group m-tile counts and their prefix. num_seq_per_group_avg only steers tile-width
// selection; update_tma is ignored. Throws std::runtime_error when the launch fails and
// std::invalid_argument for arguments the kernel cannot take.
void group_gemm_nvfp4_async(void* y_ptr, const void* x_ptr, const void* w_ptr,
                            const void* seqlens_ptr, const void* cu_seqlens_ptr,
                            const void* x_scale_ptr, const void* w_scale_ptr, void* tmas_ptr,
                            void* tiles_ptr, void* cu_tiles_ptr, int num_group, int m, int n, int k,
                            int m_scale_pad, int num_seq_per_group_avg, bool update_tma,
                            cudaStream_t stream);

// Extension without a counterpart in the reference: group_alpha[e] (FP32, may be null)
// multiplies the FP32 accumulator of group e before the FP16 rounding.
void group_gemm_nvfp4_ex_async(void* y_ptr, const void* x_ptr, const void* w_ptr,
                               const void* seqlens_ptr, const void* cu_seqlens_ptr,
                               const void* x_scale_ptr, const void* w_scale_ptr, void* tmas_ptr,
                               void* tiles_ptr, void* cu_tiles_ptr, int num_group, int m, int n,
                               int k, int m_scale_pad, int num_seq_per_group_avg, bool update_tma,
                               const float* group_alpha, cudaStream_t stream);

}  // namespace grouped_gemm
}  // namespace sm120_nvfp4
