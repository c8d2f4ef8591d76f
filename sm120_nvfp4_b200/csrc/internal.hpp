// Declarations shared between the translation units of the library (not part of the ABI).
#pragma once

#include <atomic>
#include <cstddef>

#include <cuda_runtime.h>

namespace b200 {

extern std::atomic<long long> g_launch_count;

inline void count_launch(int n = 1) { g_launch_count.fetch_add(n, std::memory_order_relaxed); }

// Status of the launch(es) just issued. cudaGetLastError, not cudaPeekAtLastError: a launch that
// was refused (bad configuration) is reported by the call that caused it and does not linger to
// fail the next, unrelated call.
inline int launch_status() { return cudaGetLastError() == cudaSuccess ? 0 : 6; }

int gemm_dense(int groups, int m, int n, int k, const void* a, const void* b, const void* sfa,
               const void* sfb, void* c, bool out_f32, cudaStream_t stream);

int gemm_splitk(int m, int n, int k, int split_k, const void* a, const void* b, const void* sfa,
                const void* sfb, void* c_f16, void* workspace, size_t workspace_bytes,
                cudaStream_t stream);

int gemm_splitk_cluster(int m, int n, int k, int split_k, const void* a, const void* b, const void* sfa,
                        const void* sfb, void* c_f16, cudaStream_t stream);

int gemm_grouped(void* y, const void* x, const void* w, const void* seqlens,
                 const void* cu_seqlens, const void* x_scale, const void* w_scale, void* tiles,
                 void* cu_tiles, int num_group, int m, int n, int k, int m_scale_pad,
                 int num_seq_per_group_avg, const float* group_alpha, cudaStream_t stream,
                 int col_start = 0, int col_count = 0);

int gemm_grouped_swiglu(void* q_out, void* q_scale, const void* x, const void* w, const void* seqlens,
                        const void* cu_seqlens, const void* x_scale, const void* w_scale, void* tiles,
                        void* cu_tiles, int num_group, int m, int inter, int k, int m_scale_pad,
                        int q_scale_m_pad, int num_seq_per_group_avg, cudaStream_t stream);

int moe_count_and_gather(void* gate_up_input, void* gate_up_input_scale, const void* input,
                         const void* input_scale, const void* topk_ids, void* topk_pos,
                         void* seqlens, void* cu_seqlens, int num_tokens, int hidden_size,
                         int num_topk, int num_expert_local, int rank_ep, int input_scale_m_pad,
                         int grouped_scale_m_pad, bool zero_scales, cudaStream_t stream);

int moe_act_mul_and_quant(void* output, void* output_scale, const void* gate_up, const void* seqlens,
                          const void* cu_seqlens, int num_expert_local, int total_rows,
                          int grouped_scale_m_pad, int intermediate_size, bool zero_scales,
                          cudaStream_t stream);

int moe_quantize_expert(void* output, void* output_scale, const void* input, const void* seqlens,
                        const void* cu_seqlens, const void* row_map, int num_expert_local,
                        int total_rows, int hidden_size, int grouped_scale_m_pad, int input_dtype,
                        bool zero_scales, cudaStream_t stream);

int moe_route(const void* topk_ids, void* topk_pos, void* seqlens, void* cu_seqlens, int num_tokens,
              int num_topk, int num_expert_local, int rank_ep, cudaStream_t stream);

int moe_move_rows(void* dst, const void* src, const void* index, int count, int fanout, int row_bytes,
                  bool scatter, cudaStream_t stream);

int moe_router_topk(const void* logits, void* topk_ids, void* topk_weights, int num_tokens,
                    int num_experts, int num_topk, cudaStream_t stream);

int moe_silu_f16(void* out_f32, const void* in_f16, int count, cudaStream_t stream);

int moe_reduce(void* output, const void* down_output, const void* topk_pos, const void* topk_scale,
               const void* shared_output, int num_tokens, int hidden_size, int num_topk,
               bool out_is_bf16, cudaStream_t stream);

}  // namespace b200
