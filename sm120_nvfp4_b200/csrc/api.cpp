// sm120_nvfp4 C++ API: translation between the C ABI's int statuses and the reference's
// conventions (GemmStatus for the GEMM family, exceptions for grouped GEMM and MoE).
#include <stdexcept>
#include <string>

#include "b200_nvfp4.h"
#include "sm120_nvfp4/fused_moe.hpp"
#include "sm120_nvfp4/gemm.hpp"
#include "sm120_nvfp4/grouped_gemm.hpp"

namespace sm120_nvfp4 {

namespace {

GemmStatus to_status(int s) { return static_cast<GemmStatus>(s); }

void throw_on_error(int status, const char* what) {
  if (status == B200_NVFP4_SUCCESS) return;
  std::string msg = std::string(what) + ": " + b200_nvfp4_status_string(status);
  if (status == B200_NVFP4_CUDA_ERROR || status == B200_NVFP4_UNSUPPORTED_DEVICE)
    throw std::runtime_error(msg);
  throw std::invalid_argument(msg);
}

}  // namespace

const char* gemm_status_string(GemmStatus status) {
  return b200_nvfp4_status_string(static_cast<int>(status));
}

const char* nvfp4_gemm_path_string(Nvfp4GemmPath path) {
  return b200_nvfp4_gemm_path_string(static_cast<int>(path));
}

Nvfp4GemmPath nvfp4_gemm_path_sm120(int m, int n, int k) {
  return static_cast<Nvfp4GemmPath>(b200_nvfp4_gemm_path(m, n, k));
}

GemmStatus nvfp4_cute_gemm_sm120(int m, int n, int k, const void* a, const void* b, const void* sfa,
                                 const void* sfb, half* c, cudaStream_t stream) {
  return to_status(b200_nvfp4_gemm(1, m, n, k, a, b, sfa, sfb, c, 0, stream));
}

GemmStatus nvfp4_cute_gemm_f32_sm120(int m, int n, int k, const void* a, const void* b,
                                     const void* sfa, const void* sfb, float* c, cudaStream_t stream) {
  return to_status(b200_nvfp4_gemm(1, m, n, k, a, b, sfa, sfb, c, 1, stream));
}

GemmStatus nvfp4_cute_batched_gemm_sm120(int groups, int m, int n, int k, const void* a,
                                         const void* b, const void* sfa, const void* sfb, half* c,
                                         cudaStream_t stream) {
  return to_status(b200_nvfp4_gemm(groups, m, n, k, a, b, sfa, sfb, c, 0, stream));
}

GemmStatus nvfp4_cute_batched_gemm_f32_sm120(int groups, int m, int n, int k, const void* a,
                                             const void* b, const void* sfa, const void* sfb,
                                             float* c, cudaStream_t stream) {
  return to_status(b200_nvfp4_gemm(groups, m, n, k, a, b, sfa, sfb, c, 1, stream));
}

std::size_t nvfp4_cutlass_gemm_workspace_size_sm120(int, int, int) { return 0; }

GemmStatus nvfp4_cutlass_gemm_sm120(int m, int n, int k, const void* a, const void* b,
                                    const void* sfa, const void* sfb, half* c, void*, std::size_t,
                                    cudaStream_t stream) {
  return nvfp4_cute_gemm_sm120(m, n, k, a, b, sfa, sfb, c, stream);
}

std::size_t nvfp4_gemm_workspace_size_sm120(int m, int n, int k) {
  return b200_nvfp4_gemm_workspace_bytes(m, n, k);
}

GemmStatus nvfp4_gemm_sm120(int m, int n, int k, const void* a, const void* b, const void* sfa,
                            const void* sfb, half* c, void* workspace, std::size_t workspace_bytes,
                            cudaStream_t stream) {
  return to_status(b200_nvfp4_gemm_auto(m, n, k, a, b, sfa, sfb, c, workspace, workspace_bytes, stream));
}

namespace grouped_gemm {

void group_gemm_nvfp4_ex_async(void* y_ptr, const void* x_ptr, const void* w_ptr,
                               const void* seqlens_ptr, const void* cu_seqlens_ptr,
                               const void* x_scale_ptr, const void* w_scale_ptr, void* tmas_ptr,
                               void* tiles_ptr, void* cu_tiles_ptr, int num_group, int m, int n,
                               int k, int m_scale_pad, int num_seq_per_group_avg, bool update_tma,
                               const float* group_alpha, cudaStream_t stream) {
  throw_on_error(b200_nvfp4_grouped_gemm(y_ptr, x_ptr, w_ptr, seqlens_ptr, cu_seqlens_ptr,
                                         x_scale_ptr, w_scale_ptr, tmas_ptr, tiles_ptr, cu_tiles_ptr,
                                         num_group, m, n, k, m_scale_pad, num_seq_per_group_avg,
                                         update_tma ? 1 : 0, group_alpha, stream),
                 "group_gemm_nvfp4");
}

void group_gemm_nvfp4_async(void* y_ptr, const void* x_ptr, const void* w_ptr,
                            const void* seqlens_ptr, const void* cu_seqlens_ptr,
                            const void* x_scale_ptr, const void* w_scale_ptr, void* tmas_ptr,
                            void* tiles_ptr, void* cu_tiles_ptr, int num_group, int m, int n, int k,
                            int m_scale_pad, int num_seq_per_group_avg, bool update_tma,
                            cudaStream_t stream) {
  group_gemm_nvfp4_ex_async(y_ptr, x_ptr, w_ptr, seqlens_ptr, cu_seqlens_ptr, x_scale_ptr,
                            w_scale_ptr, tmas_ptr, tiles_ptr, cu_tiles_ptr, num_group, m, n, k,
                            m_scale_pad, num_seq_per_group_avg, update_tma, nullptr, stream);
}

}  // namespace grouped_gemm

namespace fused_moe {

void count_and_gather_nvfp4_async(void* gate_up_input_ptr, void* gate_up_input_scale_ptr,
                                  const void* input_ptr, const void* input_scale_ptr,
                                  const void* topk_ids_ptr, void* topk_pos_ptr, void* seqlens_ptr,
                                  void* cu_seqlens_ptr, int num_tokens, int hidden_size,
                                  int num_topk, int num_expert_local, int rank_ep,
                                  int input_scale_m_pad, int grouped_scale_m_pad,
                                  cudaStream_t stream) {
  throw_on_error(b200_nvfp4_moe_count_and_gather(
                     gate_up_input_ptr, gate_up_input_scale_ptr, input_ptr, input_scale_ptr,
                     topk_ids_ptr, topk_pos_ptr, seqlens_ptr, cu_seqlens_ptr, num_tokens,
                     hidden_size, num_topk, num_expert_local, rank_ep, input_scale_m_pad,
                     grouped_scale_m_pad, /*zero_scales=*/1, stream),
                 "count_and_gather_nvfp4");
}

void act_mul_and_quant_nvfp4_async(void* output_ptr, void* output_scale_ptr,
                                   const void* gate_up_ptr, const void* seqlens_ptr,
                                   const void* cu_seqlens_ptr, int num_expert_local,
                                   int grouped_scale_m_pad, int intermediate_size,
                                   cudaStream_t stream) {
  // The reference signature carries no row count; the kernel reads it from cu_seqlens[E].
  const int rows_hint = 0;
  throw_on_error(b200_nvfp4_moe_act_mul_and_quant(output_ptr, output_scale_ptr, gate_up_ptr,
                                                  seqlens_ptr, cu_seqlens_ptr, num_expert_local,
                                                  rows_hint, grouped_scale_m_pad, intermediate_size,
                                                  /*zero_scales=*/1, stream),
                 "act_mul_and_quant_nvfp4");
}

void quantize_expert_nvfp4_async(void* output_ptr, void* output_scale_ptr, const void* input_ptr,
                                 const void* seqlens_ptr, const void* cu_seqlens_ptr,
                                 int num_expert_local, int total_rows, int hidden_size,
                                 int grouped_scale_m_pad, bool input_is_bf16, cudaStream_t stream) {
  throw_on_error(b200_nvfp4_moe_quantize_expert(output_ptr, output_scale_ptr, input_ptr, seqlens_ptr,
                                                cu_seqlens_ptr, num_expert_local, total_rows,
                                                hidden_size, grouped_scale_m_pad,
                                                input_is_bf16 ? 1 : 0, /*zero_scales=*/1, stream),
                 "quantize_expert_nvfp4");
}

void reduce_nvfp4_async(void* output_ptr, const void* down_output_ptr, const void* topk_pos_ptr,
                        const void* topk_scale_ptr, const void* shared_output_ptr, int num_tokens,
                        int hidden_size, int num_topk, cudaStream_t stream) {
  throw_on_error(b200_nvfp4_moe_reduce(output_ptr, down_output_ptr, topk_pos_ptr, topk_scale_ptr,
                                       shared_output_ptr, num_tokens, hidden_size, num_topk, 0, stream),
                 "reduce_nvfp4");
}

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
                          int input_scale_m_pad, int grouped_scale_m_pad, cudaStream_t stream) {
  throw_on_error(
      b200_nvfp4_fused_moe(output_ptr, input_ptr, input_scale_ptr, gate_up_input_ptr,
                           gate_up_input_scale_ptr, gate_up_output_ptr, gate_up_weight_ptr,
                           gate_up_weight_scale_ptr, gate_up_tmas_ptr, down_input_ptr,
                           down_input_scale_ptr, down_output_ptr, down_weight_ptr,
                           down_weight_scale_ptr, down_tmas_ptr, topk_ids_ptr, topk_scale_ptr,
                           topk_pos_ptr, seqlens_ptr, cu_seqlens_ptr, tiles_ptr, cu_tiles_ptr,
                           shared_output_ptr, num_tokens, hidden_size, intermediate_size, num_topk,
                           num_expert_total, num_expert_local, rank_ep, input_scale_m_pad,
                           grouped_scale_m_pad, stream),
      "fuse_moe_nvfp4");
}

std::size_t expert_moe_nvfp4_workspace_size(int total_rows, int hidden_size, int intermediate_size,
                                            int num_expert_local, int grouped_scale_m_pad) {
  return b200_nvfp4_expert_moe_workspace_bytes(total_rows, hidden_size, intermediate_size,
                                               num_expert_local, grouped_scale_m_pad);
}

void expert_moe_nvfp4_async(void* output_ptr, const void* input_ptr, const void* input_scale_ptr,
                            const void* gate_up_weight_ptr, const void* gate_up_weight_scale_ptr,
                            const void* down_weight_ptr, const void* down_weight_scale_ptr,
                            const void* seqlens_ptr, const void* cu_seqlens_ptr,
                            void* workspace_ptr, std::size_t workspace_bytes, int total_rows,
                            int hidden_size, int intermediate_size, int num_expert_local,
                            int grouped_scale_m_pad, cudaStream_t stream) {
  const int status = b200_nvfp4_expert_moe(
      output_ptr, input_ptr, input_scale_ptr, gate_up_weight_ptr, gate_up_weight_scale_ptr,
      down_weight_ptr, down_weight_scale_ptr, seqlens_ptr, cu_seqlens_ptr, workspace_ptr,
      workspace_bytes, total_rows, hidden_size, intermediate_size, num_expert_local,
      grouped_scale_m_pad, stream);
  if (status == B200_NVFP4_INSUFFICIENT_WORKSPACE)
    throw std::invalid_argument("expert_moe_nvfp4 workspace is null or too small");
  throw_on_error(status, "expert_moe_nvfp4");
}

}  // namespace fused_moe
}  // namespace sm120_nvfp4
