// C++ API of the fused-MoE path, source-compatible with the reference header
// include/sm120_nvfp4/fused_moe.hpp:12-80. Functions return void and throw
// std::runtime_error on CUDA launch errors and std::invalid_argument on arguments that
// cannot be served (null / too small workspace, unsupported sizes), as the reference does.
#pragma once

#include <cstddef>

#include <cuda_runtime_api.h>

namespace sm120_nvfp4 {
namespace fused_moe {

// Counts the assignments of the local experts [rank_ep*E, rank_ep*E+E), builds
// seqlens / cu_seqlens / topk_pos (-1 for remote routes) and gathers payload rows and their
// scales into expert-major order. The grouped scale buffer is zero-filled first.
void count_and_gather_nvfp4_async(void* gate_up_input_ptr, void* gate_up_input_scale_ptr,
                                  const void* input_ptr, const void* input_scale_ptr,
                                  const void* topk_ids_ptr, void* topk_pos_ptr, void* seqlens_ptr,
                                  void* cu_seqlens_ptr, int num_tokens, int hidden_size,
                                  int num_topk, int num_expert_local, int rank_ep,
                                  int input_scale_m_pad, int grouped_scale_m_pad,
                                  cudaStream_t stream);

// gate_up FP16 [rows, 2*I] -> packed E2M1 [rows, I/2] of silu(gate)*up with per-expert
// scale regions (zero-filled first).
void act_mul_and_quant_nvfp4_async(void* output_ptr, void* output_scale_ptr,
                                   const void* gate_up_ptr, const void* seqlens_ptr,
                                   const void* cu_seqlens_ptr, int num_expert_local,
                                   int grouped_scale_m_pad, int intermediate_size,
                                   cudaStream_t stream);

// FP16 / BF16 expert-major rows -> packed E2M1 with per-expert scale regions.
void quantize_expert_nvfp4_async(void* output_ptr, void* output_scale_ptr, const void* input_ptr,
                                 const void* seqlens_ptr, const void* cu_seqlens_ptr,
                                 int num_expert_local, int total_rows, int hidden_size,
                                 int grouped_scale_m_pad, bool input_is_bf16, cudaStream_t stream);

// out[t] = half(shared[t] + sum_r scale[t,r] * down[pos[t,r]]), routes with pos < 0 skipped.
void reduce_nvfp4_async(void* output_ptr, const void* down_output_ptr, const void* topk_pos_ptr,
                        const void* topk_scale_ptr, const void* shared_output_ptr, int num_tokens,
                        int hidden_size, int num_topk, cudaStream_t stream);

// Whole routed layer; all intermediates are caller-provided.
void fuse_moe_nvfp4_async(void* output_ptr, const void* input_ptr, const void* input_scale_ptr,
                          void* gate_up_input_ptr, void* gate_up_input_scale_ptr,
                          void* gate_up_output_ptr, const void* gate_up_weight_ptr,
                          const void* gate_up_weight_scale_ptr, void* gate_up_tmas_ptr,
                          void* down_input_ptr, void* down_input_scale_ptr, void* down_output_ptr,
                          const void* down_weight_ptr, const void* down_weight_scale_ptr,
                          void* down_tmas_ptr, const void* topk_ids_ptr, const void* topk_scale_ptr,
                          void* topk_pos_ptr, void* seqlens_ptr, void* cu_seqlens_ptr,
                          void* tiles_ptr, void* cu_tiles_ptr, const void* shared_output_ptr,
                          int num_tokens, int hidden_size, int intermediate_size, int num_topk,
                          int num_expert_total, int num_expert_local, int rank_ep,
                          int input_scale_m_pad, int grouped_scale_m_pad, cudaStream_t stream);

// Expert-major hand-off for dispatchers that already routed the rows: gate/up GEMM,
// SiLU*up + quant, down GEMM. Output = expanded FP16 rows, unweighted.
std::size_t expert_moe_nvfp4_workspace_size(int total_rows, int hidden_size, int intermediate_size,
                                            int num_expert_local, int grouped_scale_m_pad);

void expert_moe_nvfp4_async(void* output_ptr, const void* input_ptr, const void* input_scale_ptr,
                            const void* gate_up_weight_ptr, const void* gate_up_weight_scale_ptr,
                            const void* down_weight_ptr, const void* down_weight_scale_ptr,
                            const void* seqlens_ptr, const void* cu_seqlens_ptr,
                            void* workspace_ptr, std::size_t workspace_bytes, int total_rows,
                            int hidden_size, int intermediate_size, int num_expert_local,
                            int grouped_scale_m_pad, cudaStream_t stream);

}  // namespace fused_moe
}  // namespace sm120_nvfp4
