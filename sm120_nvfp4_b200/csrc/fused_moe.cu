// Orchestration of the fused-MoE entry points and the C ABI of the MoE functions.
//
// fuse_moe: route + gather -> gate/up grouped GEMM -> SiLU*up + NVFP4 quant -> down grouped
// GEMM -> weighted top-k combine (src/fused_moe/fused_moe.cu:25-74). expert_moe: the three
// middle stages on rows that are already expert-major, with the reference's workspace carve
// (src/fused_moe/fused_moe.cu:76-157). Every stage is enqueued on the caller's stream; no
// host synchronisation, no allocation.
#include <atomic>
#include <cstdint>

#include "host_common.hpp"
#include "internal.hpp"

namespace b200 {

namespace {

// Gate/up GEMM -> down-projection input. Two forms with the same bits: the reference's two steps
// (grouped GEMM writes the FP16 product, a second kernel reads it back for SiLU * up + the NVFP4
// quantisation), or one kernel whose epilogue does the activation and the quantisation on the
// accumulator, so that the FP16 product (256 MiB at the DeepSeek-shaped layer) never reaches
// memory and gate_up_output stays untouched. b200_nvfp4_set_fused_gate_up chooses; the fused form
// needs an intermediate size that is a multiple of 128 and falls back to the two steps otherwise.
std::atomic<int> g_fused_gate_up{1};

int gate_up_stage(void* down_input, void* down_input_scale, void* gate_up_output, const void* x,
                  const void* w, const void* seqlens, const void* cu_seqlens, const void* x_scale,
                  const void* w_scale, void* tiles, void* cu_tiles, int num_expert_local, int total_rows,
                  int intermediate_size, int hidden_size, int m_pad, int avg, cudaStream_t stream) {
  if (g_fused_gate_up.load(std::memory_order_relaxed) != 0) {
    const int st = gemm_grouped_swiglu(down_input, down_input_scale, x, w, seqlens, cu_seqlens, x_scale, w_scale,
                                       tiles, cu_tiles, num_expert_local, total_rows, intermediate_size,
                                       hidden_size, m_pad, m_pad, avg, stream);
    if (st != B200_NVFP4_CUTLASS_NOT_SUPPORTED) return st;
  }
  int st = gemm_grouped(gate_up_output, x, w, seqlens, cu_seqlens, x_scale, w_scale, tiles, cu_tiles,
                        num_expert_local, total_rows, intermediate_size * 2, hidden_size, m_pad, avg, nullptr,
                        stream);
  if (st != B200_NVFP4_SUCCESS) return st;
  return moe_act_mul_and_quant(down_input, down_input_scale, gate_up_output, seqlens, cu_seqlens,
                               num_expert_local, total_rows, m_pad, intermediate_size,
                               /*zero_scales=*/false, stream);
}

constexpr size_t kWorkspaceAlignment = 256;

size_t align_workspace(size_t v) {
  return (v + kWorkspaceAlignment - 1) / kWorkspaceAlignment * kWorkspaceAlignment;
}

struct ExpertMoeCarve {
  size_t gate_up_output, down_input, down_input_scale, gate_up_tmas, down_tmas, tiles, cu_tiles, total;
};

// Same order, sizes and 256-byte alignment as the reference (fused_moe.cu:76-95,112-136).
ExpertMoeCarve carve(int total_rows, int intermediate_size, int num_expert_local, int m_pad) {
  ExpertMoeCarve c{};
  size_t offset = 0;
  auto take = [&offset](size_t bytes) {
    offset = align_workspace(offset);
    size_t at = offset;
    offset += bytes;
    return at;
  };
  c.gate_up_output = take(static_cast<size_t>(total_rows) * intermediate_size * 2 * sizeof(uint16_t));
  c.down_input = take(static_cast<size_t>(total_rows) * intermediate_size / 2);
  c.down_input_scale = take(static_cast<size_t>(num_expert_local) * m_pad *
                            static_cast<size_t>(scale_k_padded(intermediate_size)));
  c.gate_up_tmas = take(static_cast<size_t>(num_expert_local * 3 + 2) * 128);
  c.down_tmas = take(static_cast<size_t>(num_expert_local * 3 + 2) * 128);
  c.tiles = take(static_cast<size_t>(num_expert_local) * sizeof(int));
  c.cu_tiles = take(static_cast<size_t>(num_expert_local + 1) * sizeof(int));
  c.total = align_workspace(offset);
  return c;
}

}  // namespace

int fused_moe(void* output, const void* input, const void* input_scale, void* gate_up_input,
              void* gate_up_input_scale, void* gate_up_output, const void* gate_up_weight,
              const void* gate_up_weight_scale, void* down_input, void* down_input_scale,
              void* down_output, const void* down_weight, const void* down_weight_scale,
              const void* topk_ids, const void* topk_scale, void* topk_pos, void* seqlens,
              void* cu_seqlens, void* tiles, void* cu_tiles, const void* shared_output,
              int num_tokens, int hidden_size, int intermediate_size, int num_topk,
              int num_expert_total, int num_expert_local, int rank_ep, int input_scale_m_pad,
              int grouped_scale_m_pad, cudaStream_t stream) {
  if (num_expert_total <= 0 || num_tokens <= 0 || num_topk <= 0) return B200_NVFP4_INVALID_ARGUMENT;
  const long long total64 = static_cast<long long>(num_tokens) * num_topk;
  if (total64 > 0x7fffffffLL) return B200_NVFP4_INVALID_ARGUMENT;
  const int total = static_cast<int>(total64);
  const int avg = total / num_expert_total;
  int st = moe_count_and_gather(gate_up_input, gate_up_input_scale, input, input_scale, topk_ids,
                                topk_pos, seqlens, cu_seqlens, num_tokens, hidden_size, num_topk,
                                num_expert_local, rank_ep, input_scale_m_pad, grouped_scale_m_pad,
                                /*zero_scales=*/false, stream);
  if (st != B200_NVFP4_SUCCESS) return st;
  st = gate_up_stage(down_input, down_input_scale, gate_up_output, gate_up_input, gate_up_weight, seqlens,
                     cu_seqlens, gate_up_input_scale, gate_up_weight_scale, tiles, cu_tiles, num_expert_local,
                     total, intermediate_size, hidden_size, grouped_scale_m_pad, avg, stream);
  if (st != B200_NVFP4_SUCCESS) return st;
  st = gemm_grouped(down_output, down_input, down_weight, seqlens, cu_seqlens, down_input_scale,
                    down_weight_scale, tiles, cu_tiles, num_expert_local, total, hidden_size,
                    intermediate_size, grouped_scale_m_pad, avg, nullptr, stream);
  if (st != B200_NVFP4_SUCCESS) return st;
  return moe_reduce(output, down_output, topk_pos, topk_scale, shared_output, num_tokens,
                    hidden_size, num_topk, /*out_is_bf16=*/false, stream);
}

int expert_moe(void* output, const void* input, const void* input_scale, const void* gate_up_weight,
               const void* gate_up_weight_scale, const void* down_weight,
               const void* down_weight_scale, const void* seqlens, const void* cu_seqlens,
               void* workspace, size_t workspace_bytes, int total_rows, int hidden_size,
               int intermediate_size, int num_expert_local, int grouped_scale_m_pad,
               cudaStream_t stream) {
  if (total_rows <= 0 || num_expert_local <= 0 || intermediate_size <= 0 || hidden_size <= 0)
    return B200_NVFP4_INVALID_ARGUMENT;
  const ExpertMoeCarve c = carve(total_rows, intermediate_size, num_expert_local, grouped_scale_m_pad);
  if (workspace == nullptr || workspace_bytes < c.total) return B200_NVFP4_INSUFFICIENT_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(workspace) % kWorkspaceAlignment) != 0)
    return B200_NVFP4_INVALID_ARGUMENT;
  uint8_t* base = static_cast<uint8_t*>(workspace);
  void* gate_up_output = base + c.gate_up_output;
  void* down_input = base + c.down_input;
  void* down_input_scale = base + c.down_input_scale;
  void* tiles = base + c.tiles;
  void* cu_tiles = base + c.cu_tiles;
  const int avg = total_rows / num_expert_local;
  int st = gate_up_stage(down_input, down_input_scale, gate_up_output, input, gate_up_weight, seqlens,
                         cu_seqlens, input_scale, gate_up_weight_scale, tiles, cu_tiles, num_expert_local,
                         total_rows, intermediate_size, hidden_size, grouped_scale_m_pad, avg, stream);
  if (st != B200_NVFP4_SUCCESS) return st;
  return gemm_grouped(output, down_input, down_weight, seqlens, cu_seqlens, down_input_scale,
                      down_weight_scale, tiles, cu_tiles, num_expert_local, total_rows, hidden_size,
                      intermediate_size, grouped_scale_m_pad, avg, nullptr, stream);
}

size_t expert_moe_workspace_bytes(int total_rows, int intermediate_size, int num_expert_local,
                                  int grouped_scale_m_pad) {
  return carve(total_rows, intermediate_size, num_expert_local, grouped_scale_m_pad).total;
}

}  // namespace b200

extern "C" {

int b200_nvfp4_moe_count_and_gather(void* gate_up_input, void* gate_up_input_scale,
                                    const void* input, const void* input_scale,
                                    const void* topk_ids, void* topk_pos, void* seqlens,
                                    void* cu_seqlens, int num_tokens, int hidden_size, int num_topk,
                                    int num_expert_local, int rank_ep, int input_scale_m_pad,
                                    int grouped_scale_m_pad, int zero_scales, b200_stream_t stream) {
  return b200::moe_count_and_gather(gate_up_input, gate_up_input_scale, input, input_scale, topk_ids,
                                    topk_pos, seqlens, cu_seqlens, num_tokens, hidden_size, num_topk,
                                    num_expert_local, rank_ep, input_scale_m_pad, grouped_scale_m_pad,
                                    zero_scales != 0, static_cast<cudaStream_t>(stream));
}

int b200_nvfp4_moe_act_mul_and_quant(void* output, void* output_scale, const void* gate_up,
                                     const void* seqlens, const void* cu_seqlens,
                                     int num_expert_local, int total_rows, int grouped_scale_m_pad,
                                     int intermediate_size, int zero_scales, b200_stream_t stream) {
  return b200::moe_act_mul_and_quant(output, output_scale, gate_up, seqlens, cu_seqlens,
                                     num_expert_local, total_rows, grouped_scale_m_pad,
                                     intermediate_size, zero_scales != 0,
                                     static_cast<cudaStream_t>(stream));
}

int b200_nvfp4_moe_quantize_expert(void* output, void* output_scale, const void* input,
                                   const void* seqlens, const void* cu_seqlens, int num_expert_local,
                                   int total_rows, int hidden_size, int grouped_scale_m_pad,
                                   int input_is_bf16, int zero_scales, b200_stream_t stream) {
  return b200::moe_quantize_expert(output, output_scale, input, seqlens, cu_seqlens, nullptr,
                                   num_expert_local, total_rows, hidden_size, grouped_scale_m_pad,
                                   input_is_bf16, zero_scales != 0,
                                   static_cast<cudaStream_t>(stream));
}

int b200_nvfp4_moe_quantize_expert_gather(void* output, void* output_scale, const void* input,
                                          const void* row_map, const void* seqlens,
                                          const void* cu_seqlens, int num_expert_local, int total_rows,
                                          int hidden_size, int grouped_scale_m_pad, int input_is_bf16,
                                          int zero_scales, b200_stream_t stream) {
  return b200::moe_quantize_expert(output, output_scale, input, seqlens, cu_seqlens, row_map,
                                   num_expert_local, total_rows, hidden_size, grouped_scale_m_pad,
                                   input_is_bf16, zero_scales != 0,
                                   static_cast<cudaStream_t>(stream));
}

int b200_nvfp4_moe_route(const void* topk_ids, void* topk_pos, void* seqlens, void* cu_seqlens,
                         int num_tokens, int num_topk, int num_expert_local, int rank_ep,
                         b200_stream_t stream) {
  return b200::moe_route(topk_ids, topk_pos, seqlens, cu_seqlens, num_tokens, num_topk,
                         num_expert_local, rank_ep, static_cast<cudaStream_t>(stream));
}

int b200_nvfp4_moe_scatter_rows(void* dst, const void* src, const void* pos, int count, int fanout,
                                int row_bytes, b200_stream_t stream) {
  return b200::moe_move_rows(dst, src, pos, count, fanout, row_bytes, true,
                             static_cast<cudaStream_t>(stream));
}

int b200_nvfp4_moe_gather_rows(void* dst, const void* src, const void* map, int count, int row_bytes,
                               b200_stream_t stream) {
  return b200::moe_move_rows(dst, src, map, count, 1, row_bytes, false,
                             static_cast<cudaStream_t>(stream));
}

int b200_nvfp4_moe_reduce(void* output, const void* down_output, const void* topk_pos,
                          const void* topk_scale, const void* shared_output, int num_tokens,
                          int hidden_size, int num_topk, int out_is_bf16, b200_stream_t stream) {
  return b200::moe_reduce(output, down_output, topk_pos, topk_scale, shared_output, num_tokens,
                          hidden_size, num_topk, out_is_bf16 != 0, static_cast<cudaStream_t>(stream));
}

int b200_nvfp4_fused_moe(void* output, const void* input, const void* input_scale,
                         void* gate_up_input, void* gate_up_input_scale, void* gate_up_output,
                         const void* gate_up_weight, const void* gate_up_weight_scale,
                         void* gate_up_tmas, void* down_input, void* down_input_scale,
                         void* down_output, const void* down_weight, const void* down_weight_scale,
                         void* down_tmas, const void* topk_ids, const void* topk_scale,
                         void* topk_pos, void* seqlens, void* cu_seqlens, void* tiles, void* cu_tiles,
                         const void* shared_output, int num_tokens, int hidden_size,
                         int intermediate_size, int num_topk, int num_expert_total,
                         int num_expert_local, int rank_ep, int input_scale_m_pad,
                         int grouped_scale_m_pad, b200_stream_t stream) {
  (void)gate_up_tmas;
  (void)down_tmas;
  return b200::fused_moe(output, input, input_scale, gate_up_input, gate_up_input_scale,
                         gate_up_output, gate_up_weight, gate_up_weight_scale, down_input,
                         down_input_scale, down_output, down_weight, down_weight_scale, topk_ids,
                         topk_scale, topk_pos, seqlens, cu_seqlens, tiles, cu_tiles, shared_output,
                         num_tokens, hidden_size, intermediate_size, num_topk, num_expert_total,
                         num_expert_local, rank_ep, input_scale_m_pad, grouped_scale_m_pad,
                         static_cast<cudaStream_t>(stream));
}

int b200_nvfp4_grouped_gemm_swiglu_quant(void* output, void* output_scale, const void* x, const void* w,
                                         const void* seqlens, const void* cu_seqlens, const void* x_scale,
                                         const void* w_scale, void* tiles, void* cu_tiles, int num_group, int m,
                                         int intermediate_size, int k, int m_scale_pad, int output_scale_m_pad,
                                         int num_seq_per_group_avg, b200_stream_t stream) {
  return b200::gemm_grouped_swiglu(output, output_scale, x, w, seqlens, cu_seqlens, x_scale, w_scale, tiles,
                                   cu_tiles, num_group, m, intermediate_size, k, m_scale_pad, output_scale_m_pad,
                                   num_seq_per_group_avg, static_cast<cudaStream_t>(stream));
}

int b200_nvfp4_moe_router_topk(const void* logits, void* topk_ids, void* topk_weights,
                               int num_tokens, int num_experts, int num_topk, b200_stream_t stream) {
  return b200::moe_router_topk(logits, topk_ids, topk_weights, num_tokens, num_experts, num_topk,
                               static_cast<cudaStream_t>(stream));
}

size_t b200_nvfp4_expert_moe_workspace_bytes(int total_rows, int hidden_size, int intermediate_size,
                                             int num_expert_local, int grouped_scale_m_pad) {
  (void)hidden_size;
  return b200::expert_moe_workspace_bytes(total_rows, intermediate_size, num_expert_local,
                                          grouped_scale_m_pad);
}

int b200_nvfp4_expert_moe(void* output, const void* input, const void* input_scale,
                          const void* gate_up_weight, const void* gate_up_weight_scale,
                          const void* down_weight, const void* down_weight_scale, const void* seqlens,
                          const void* cu_seqlens, void* workspace, size_t workspace_bytes,
                          int total_rows, int hidden_size, int intermediate_size,
                          int num_expert_local, int grouped_scale_m_pad, b200_stream_t stream) {
  return b200::expert_moe(output, input, input_scale, gate_up_weight, gate_up_weight_scale,
                          down_weight, down_weight_scale, seqlens, cu_seqlens, workspace,
                          workspace_bytes, total_rows, hidden_size, intermediate_size,
                          num_expert_local, grouped_scale_m_pad, static_cast<cudaStream_t>(stream));
}

int b200_nvfp4_silu_f16(void* out_f32, const void* in_f16, int count, b200_stream_t stream) {
  return b200::moe_silu_f16(out_f32, in_f16, count, static_cast<cudaStream_t>(stream));
}

int b200_nvfp4_set_fused_gate_up(int enabled) {
  b200::g_fused_gate_up.store(enabled != 0 ? 1 : 0, std::memory_order_relaxed);
  return B200_NVFP4_SUCCESS;
}

}  // extern "C"
