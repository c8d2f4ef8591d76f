/*
 * C ABI of the B200 (sm_100a) NVFP4 GEMM / grouped GEMM / fused-MoE library.
 *
 * Every entry point takes plain device pointers, integer sizes and a CUDA stream
 * (cudaStream_t, i.e. an opaque pointer; NULL = the default stream), enqueues work on that
 * stream and returns at once with an int status (B200_NVFP4_* below). Nothing here
 * allocates or frees device memory or synchronises, unless a comment says otherwise.
 * These are the functions a foreign-function binding (ctypes, cgo, JNI, ...) binds; the
 * C++ API in include/sm120_nvfp4/ is a thin wrapper over them.
 *
 * Data formats (same as the reference, include/sm120_nvfp4/gemm.hpp:13-54):
 *   payload  packed E2M1, two values per byte, low nibble = even k, K contiguous;
 *   scales   raw UE4M3 bytes, one per 16 consecutive K values, stored in 512-byte atoms
 *            (128 rows x 4 k-blocks): offset(row, kb) = ((row/128)*ceil(K/64) + kb/4)*512
 *            + (row%32)*16 + ((row%128)/32)*4 + kb%4; a region holds
 *            align128(rows) * align4(ceil(K/16)) bytes and must be 16-byte aligned;
 *   outputs  row-major FP16 (or FP32 where stated).
 * Shape rules: M, N, K > 0, K % 32 == 0, N % 8 == 0 (src/gemm/cute_gemm.cu:351-355).
 */
#ifndef B200_NVFP4_H_
#define B200_NVFP4_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef B200_NVFP4_API
#define B200_NVFP4_API __attribute__((visibility("default")))
#endif

/* Status codes. 0..6 have the values and order of sm120_nvfp4::GemmStatus
 * (include/sm120_nvfp4/gemm.hpp:56-64). */
enum {
  B200_NVFP4_SUCCESS = 0,
  B200_NVFP4_INVALID_ARGUMENT = 1,
  B200_NVFP4_UNSUPPORTED_DEVICE = 2,
  B200_NVFP4_INSUFFICIENT_WORKSPACE = 3,
  B200_NVFP4_CUTLASS_NOT_SUPPORTED = 4,
  B200_NVFP4_CUTLASS_ERROR = 5,
  B200_NVFP4_CUDA_ERROR = 6
};

/* Paths of the default dispatcher: values of sm120_nvfp4::Nvfp4GemmPath (gemm.hpp:70-74). */
enum { B200_NVFP4_PATH_GENERIC = 0, B200_NVFP4_PATH_M128_SPLITK4 = 1, B200_NVFP4_PATH_M256_SPLITK2 = 2 };

typedef void* b200_stream_t; /* a cudaStream_t */

/* gemm_status_string (src/gemm/status.cpp:5-23), for every status above. */
B200_NVFP4_API const char* b200_nvfp4_status_string(int status);

/* nvfp4_gemm_path_string (src/gemm/gemm_dispatch.cu:32-42). */
B200_NVFP4_API const char* b200_nvfp4_gemm_path_string(int path);

/* nvfp4_gemm_path_sm120 (src/gemm/gemm_dispatch.cu:44-56): deterministic, does not look
 * at the device. M == 128 -> split-K 4, M == 256 -> split-K 2 when K % 32 == 0,
 * N % 8 == 0 and ceil(K/128) >= split; otherwise the generic path. */
B200_NVFP4_API int b200_nvfp4_gemm_path(int m, int n, int k);

/* nvfp4_gemm_workspace_size_sm120 (src/gemm/gemm_dispatch.cu:58-61):
 * split * M * N * 4 bytes for the two split-K paths, else 0. */
B200_NVFP4_API size_t b200_nvfp4_gemm_workspace_bytes(int m, int n, int k);

/* nvfp4_cute_gemm_sm120 / nvfp4_cute_gemm_f32_sm120 / nvfp4_cute_batched_gemm(_f32)_sm120
 * (include/sm120_nvfp4/gemm.hpp:86-113, src/gemm/cute_gemm.cu:357-466).
 * C[g] = (A[g] * SFA[g]) (B[g] * SFB[g])^T for g < groups; operands contiguous
 * [groups, M, K/2], [groups, N, K/2], outputs [groups, M, N]; one scale region per group.
 * out_is_f32 selects FP32 output (the FP32 accumulator, not narrowed). */
B200_NVFP4_API int b200_nvfp4_gemm(int groups, int m, int n, int k, const void* a, const void* b,
                                   const void* sfa, const void* sfb, void* c, int out_is_f32,
                                   b200_stream_t stream);

/* gemm_specialized::m128::launch / m256::launch
 * (src/gemm/specialized/m128_gemm.cu:417-518): split-K partial sums as FP32
 * [split_k, M, N] in `workspace`, then C = half(sum over splits, in split order).
 * Any M is accepted here; the dispatcher only routes M == 128 / 256 to it. */
B200_NVFP4_API int b200_nvfp4_gemm_splitk(int m, int n, int k, int split_k, const void* a,
                                          const void* b, const void* sfa, const void* sfb,
                                          void* c_f16, void* workspace, size_t workspace_bytes,
                                          b200_stream_t stream);

/* The same split-K GEMM with the partial tiles reduced on the chip (no counterpart in the
 * reference): the split_k (2 or 4) CTAs of a cluster compute the K ranges b200_nvfp4_gemm_splitk
 * uses, exchange the FP32 partial tiles through distributed shared memory, add them in split order
 * and round once to FP16 - the bits of b200_nvfp4_gemm_splitk on the same operands - in one launch,
 * without a workspace and without a round trip of partial sums through HBM. The default dispatcher
 * uses it for its M == 128 / 256 paths. */
B200_NVFP4_API int b200_nvfp4_gemm_splitk_cluster(int m, int n, int k, int split_k, const void* a,
                                                  const void* b, const void* sfa, const void* sfb,
                                                  void* c_f16, b200_stream_t stream);

/* Split-K GEMM for callers that cannot hand over a workspace and must not allocate one: a
 * plugin hook that receives only operand pointers and a stream, a runtime whose memory plan
 * is frozen, a serving loop that may not touch the device allocator (an allocation can
 * synchronise the device). Same arithmetic and result as b200_nvfp4_gemm_splitk; the FP32
 * partial sums go to a fixed 16 MiB array in the library's device data segment, so the call
 * allocates nothing. No counterpart in the reference.
 *   - split_k * M * N must not exceed b200_nvfp4_gemm_splitk_static_max_elements() (4 Mi);
 *     beyond it the call returns B200_NVFP4_INSUFFICIENT_WORKSPACE and launches nothing.
 *   - one array per device: calls that overlap in time on the same device race on it;
 *     keep them on one stream or order them with events.
 *   - the first call on each device looks the array's address up on the host; make it before
 *     starting any stream capture.
 *   - the array needs no clearing between calls. */
B200_NVFP4_API size_t b200_nvfp4_gemm_splitk_static_max_elements(void);
B200_NVFP4_API int b200_nvfp4_gemm_splitk_static(int m, int n, int k, int split_k, const void* a,
                                                 const void* b, const void* sfa, const void* sfb,
                                                 void* c_f16, b200_stream_t stream);

/* GEMM on operands in host memory, C_host = A_host x B_host^T (FP16), with the copies in both
 * directions overlapped with the arithmetic: A and B are uploaded in chunks of block_rows /
 * block_cols rows (alternately), the block of C that a pair of chunks completes is computed as
 * soon as both have landed and copied home while later chunks still arrive. No counterpart in
 * the reference, whose entry points take device pointers only; it serves callers whose data
 * starts and ends on the host, for whom the copies, not the kernel, are the cost.
 *   - *_host: the same layouts as b200_nvfp4_gemm's operands, in host memory (page-locked
 *     memory lets the copies run asynchronously and overlap);
 *   - *_dev: device scratch of the same sizes (A m*k/2, B n*k/2, the two scale regions,
 *     C m*n*2 bytes); the library allocates none. C's scratch holds blocks, not a matrix.
 *   - block_rows, block_cols: multiples of 128, 0 for the defaults (2048, 2048); at most 64
 *     chunks per operand;
 *   - everything is enqueued; `stream` waits for the last copy, so synchronising `stream`
 *     is enough before reading c_host_f16. Calls on one device are serialised on the host. */
B200_NVFP4_API int b200_nvfp4_gemm_host(int m, int n, int k, const void* a_host, const void* b_host,
                                        const void* sfa_host, const void* sfb_host, void* c_host_f16,
                                        void* a_dev, void* b_dev, void* sfa_dev, void* sfb_dev,
                                        void* c_dev, int block_rows, int block_cols,
                                        b200_stream_t stream);

/* nvfp4_gemm_sm120 (src/gemm/gemm_dispatch.cu:63-90): default dispatcher. The M == 128 / 256 paths
 * require the workspace of b200_nvfp4_gemm_workspace_bytes as the reference does (status 3 without
 * it) and compute the split-K result on chip (b200_nvfp4_gemm_splitk_cluster, same bits). */
B200_NVFP4_API int b200_nvfp4_gemm_auto(int m, int n, int k, const void* a, const void* b,
                                        const void* sfa, const void* sfb, void* c_f16,
                                        void* workspace, size_t workspace_bytes,
                                        b200_stream_t stream);

/* grouped_gemm::group_gemm_nvfp4_async (include/sm120_nvfp4/grouped_gemm.hpp:15-21,
 * src/grouped_gemm/grouped_gemm.cu:124-144). Rows of group e are
 * [cu_seqlens[e], cu_seqlens[e] + seqlens[e]) of x [m, K/2]; w is [G, N, K/2]; x_scale has
 * one region of m_scale_pad * align4(K/16) bytes per group, indexed by the row inside the
 * group; w_scale one region of align128(N) * align4(K/16) bytes per group. y is FP16
 * [m, N]; rows that belong to no group are not written. tmas / tiles / cu_tiles are the
 * reference's per-call scratch: tmas is unused here (may be NULL), tiles [G] and
 * cu_tiles [G+1] are filled when non-NULL. num_seq_per_group_avg is a scheduling hint only;
 * update_tma is ignored as in the reference. group_alpha (may be NULL) is an extension with
 * no counterpart in the reference ABI: one FP32 multiplier per group applied to the FP32
 * accumulator before the FP16 rounding. G <= 1024. */
B200_NVFP4_API int b200_nvfp4_grouped_gemm(void* y, const void* x, const void* w,
                                           const void* seqlens, const void* cu_seqlens,
                                           const void* x_scale, const void* w_scale, void* tmas,
                                           void* tiles, void* cu_tiles, int num_group, int m,
                                           int n, int k, int m_scale_pad,
                                           int num_seq_per_group_avg, int update_tma,
                                           const float* group_alpha, b200_stream_t stream);

/* b200_nvfp4_grouped_gemm restricted to the output columns [col_start, col_start + col_count) of
 * the full [m, N] product (no counterpart in the reference): y, w and w_scale are the same whole
 * arrays as in the full call, only that column block of y is written, with the same bits as the
 * full call writes there. col_start is a multiple of 128; col_count a multiple of 128 unless the
 * window ends at N. Lets a caller pipeline the consumer of y against the rest of the product. */
B200_NVFP4_API int b200_nvfp4_grouped_gemm_columns(void* y, const void* x, const void* w,
                                                   const void* seqlens, const void* cu_seqlens,
                                                   const void* x_scale, const void* w_scale,
                                                   int num_group, int m, int n, int k, int m_scale_pad,
                                                   int num_seq_per_group_avg, const float* group_alpha,
                                                   int col_start, int col_count, b200_stream_t stream);

/* fused_moe::count_and_gather_nvfp4_async (include/sm120_nvfp4/fused_moe.hpp:12-20,
 * src/fused_moe/count_and_gather.cu:96-143). Slots inside an expert are assigned in
 * ascending flat assignment index t * num_topk + r (the reference leaves the order to
 * atomics). zero_scales != 0 reproduces the reference's memset of the whole grouped scale
 * buffer; 0 skips it (the fused entry points use 0: rows past seqlens[e] are never read
 * into a stored result). */
B200_NVFP4_API int b200_nvfp4_moe_count_and_gather(
    void* gate_up_input, void* gate_up_input_scale, const void* input, const void* input_scale,
    const void* topk_ids, void* topk_pos, void* seqlens, void* cu_seqlens, int num_tokens,
    int hidden_size, int num_topk, int num_expert_local, int rank_ep, int input_scale_m_pad,
    int grouped_scale_m_pad, int zero_scales, b200_stream_t stream);

/* fused_moe::act_mul_and_quant_nvfp4_async (fused_moe.hpp:25-30,
 * src/fused_moe/activation.cu:170-195): silu(gate) * up -> NVFP4. total_rows bounds the
 * rows of gate_up and only sizes the grid (0 = unknown); the live row count is read from
 * cu_seqlens[E] on the device. zero_scales as above. */
B200_NVFP4_API int b200_nvfp4_moe_act_mul_and_quant(void* output, void* output_scale,
                                                    const void* gate_up, const void* seqlens,
                                                    const void* cu_seqlens, int num_expert_local,
                                                    int total_rows, int grouped_scale_m_pad,
                                                    int intermediate_size, int zero_scales,
                                                    b200_stream_t stream);

/* fused_moe::quantize_expert_nvfp4_async (fused_moe.hpp:35-39,
 * src/fused_moe/activation.cu:197-232): FP16 / BF16 rows -> NVFP4, expert-major.
 * input_is_bf16: 0 = FP16, 1 = BF16 (the reference's two types), 2 = FP32 rows (an addition, for
 * packing weights from FP32 or dequantised FP8 checkpoints without an intermediate rounding). */
B200_NVFP4_API int b200_nvfp4_moe_quantize_expert(void* output, void* output_scale,
                                                  const void* input, const void* seqlens,
                                                  const void* cu_seqlens, int num_expert_local,
                                                  int total_rows, int hidden_size,
                                                  int grouped_scale_m_pad, int input_is_bf16,
                                                  int zero_scales, b200_stream_t stream);

/* Extension (no counterpart in the reference): quantize_expert that also permutes - grouped
 * row r is read from input row row_map[r] (int32, may be NULL = identity). Used by the
 * expert-parallel driver to turn rows received source-major into expert-major NVFP4 in one
 * pass. */
B200_NVFP4_API int b200_nvfp4_moe_quantize_expert_gather(void* output, void* output_scale,
                                                         const void* input, const void* row_map,
                                                         const void* seqlens, const void* cu_seqlens,
                                                         int num_expert_local, int total_rows,
                                                         int hidden_size, int grouped_scale_m_pad,
                                                         int input_is_bf16, int zero_scales,
                                                         b200_stream_t stream);

/* Extension: the routing half of count_and_gather alone (src/fused_moe/count_and_gather.cu:
 * 12-38 plus the slot assignment of :59-64, made deterministic): seqlens[E], cu_seqlens[E+1]
 * and topk_pos (grouped row of every assignment, -1 for experts outside
 * [rank_ep*E, rank_ep*E+E)). */
B200_NVFP4_API int b200_nvfp4_moe_route(const void* topk_ids, void* topk_pos, void* seqlens,
                                        void* cu_seqlens, int num_tokens, int num_topk,
                                        int num_expert_local, int rank_ep, b200_stream_t stream);

/* Extension: row movers of the expert-parallel dispatch / combine (rows of row_bytes bytes,
 * row_bytes % 16 == 0). scatter: dst[pos[a]] = src[a / fanout] for a < count, pos[a] >= 0.
 * gather: dst[i] = src[map[i]] for i < count, map[i] >= 0. */
B200_NVFP4_API int b200_nvfp4_moe_scatter_rows(void* dst, const void* src, const void* pos, int count,
                                               int fanout, int row_bytes, b200_stream_t stream);
B200_NVFP4_API int b200_nvfp4_moe_gather_rows(void* dst, const void* src, const void* map, int count,
                                              int row_bytes, b200_stream_t stream);

/* fused_moe::reduce_nvfp4_async (fused_moe.hpp:41-45, src/fused_moe/reduce.cu:39-55):
 * out[t] = half(shared[t] + sum_r w[t,r] * down[pos[t,r]]) in FP32, route order, skipping
 * pos < 0. out_is_bf16 != 0 (extension) rounds the same FP32 sum to BF16 instead. */
B200_NVFP4_API int b200_nvfp4_moe_reduce(void* output, const void* down_output,
                                         const void* topk_pos, const void* topk_scale,
                                         const void* shared_output, int num_tokens,
                                         int hidden_size, int num_topk, int out_is_bf16,
                                         b200_stream_t stream);

/* fused_moe::fuse_moe_nvfp4_async (fused_moe.hpp:49-63, src/fused_moe/fused_moe.cu:25-74).
 * Same argument list and meaning; every intermediate is caller memory. */
B200_NVFP4_API int b200_nvfp4_fused_moe(
    void* output, const void* input, const void* input_scale, void* gate_up_input,
    void* gate_up_input_scale, void* gate_up_output, const void* gate_up_weight,
    const void* gate_up_weight_scale, void* gate_up_tmas, void* down_input,
    void* down_input_scale, void* down_output, const void* down_weight,
    const void* down_weight_scale, void* down_tmas, const void* topk_ids, const void* topk_scale,
    void* topk_pos, void* seqlens, void* cu_seqlens, void* tiles, void* cu_tiles,
    const void* shared_output, int num_tokens, int hidden_size, int intermediate_size,
    int num_topk, int num_expert_total, int num_expert_local, int rank_ep,
    int input_scale_m_pad, int grouped_scale_m_pad, b200_stream_t stream);

/* fused_moe::expert_moe_nvfp4_workspace_size (fused_moe.hpp:69-71,
 * src/fused_moe/fused_moe.cu:76-95): same carve order and 256-byte alignment. */
B200_NVFP4_API size_t b200_nvfp4_expert_moe_workspace_bytes(int total_rows, int hidden_size,
                                                            int intermediate_size,
                                                            int num_expert_local,
                                                            int grouped_scale_m_pad);

/* fused_moe::expert_moe_nvfp4_async (fused_moe.hpp:73-80, src/fused_moe/fused_moe.cu:97-157).
 * Returns B200_NVFP4_INSUFFICIENT_WORKSPACE where the reference throws
 * std::invalid_argument. */
B200_NVFP4_API int b200_nvfp4_expert_moe(void* output, const void* input, const void* input_scale,
                                         const void* gate_up_weight,
                                         const void* gate_up_weight_scale,
                                         const void* down_weight, const void* down_weight_scale,
                                         const void* seqlens, const void* cu_seqlens,
                                         void* workspace, size_t workspace_bytes, int total_rows,
                                         int hidden_size, int intermediate_size,
                                         int num_expert_local, int grouped_scale_m_pad,
                                         b200_stream_t stream);

/* Gate/up grouped GEMM with SiLU(gate) * up and the NVFP4 quantisation fused into its epilogue
 * (no counterpart in the reference, which runs group_gemm_nvfp4_async and
 * act_mul_and_quant_nvfp4_async one after the other, src/fused_moe/fused_moe.cu:52-63; the fused
 * MoE entry points of this library use this kernel unless b200_nvfp4_set_fused_gate_up(0) was
 * called). w is [G, 2I, K/2] with the gate rows first;
 * output is packed E2M1 [m, I/2], output_scale one region of output_scale_m_pad rows per group -
 * the bytes the two separate calls produce. intermediate_size must be a multiple of 128
 * (otherwise B200_NVFP4_CUTLASS_NOT_SUPPORTED is returned and nothing is launched). tiles /
 * cu_tiles as in b200_nvfp4_grouped_gemm (may be null). */
B200_NVFP4_API int b200_nvfp4_grouped_gemm_swiglu_quant(
    void* output, void* output_scale, const void* x, const void* w, const void* seqlens,
    const void* cu_seqlens, const void* x_scale, const void* w_scale, void* tiles, void* cu_tiles,
    int num_group, int m, int intermediate_size, int k, int m_scale_pad, int output_scale_m_pad,
    int num_seq_per_group_avg, b200_stream_t stream);

/* Router step in front of the routed layer (no counterpart in the reference library, whose
 * entry points take topk_ids / topk_weights as inputs): logits FP32 [T, E] -> sigmoid scores,
 * the num_topk largest per token (ties to the lower expert id) as int32 ids [T, k], and FP32
 * weights [T, k] = score / sum of the selected scores. E <= 4096. */
B200_NVFP4_API int b200_nvfp4_moe_router_topk(const void* logits, void* topk_ids,
                                              void* topk_weights, int num_tokens, int num_experts,
                                              int num_topk, b200_stream_t stream);

/* Expert-parallel hand-off (no counterpart in the reference library; its hand-off benchmark
 * benchmarks/integration/benchmark_deepep_handoff.py:356-364 ships one BF16 row per
 * (token, expert) with torch ops). A token is sent once to each rank that owns one of its
 * experts, as a wire record
 *   [payload H/2 | UE4M3 scales H/16 in k-block order | ids k x int32 | weights k x float]
 * padded to 16 bytes; hidden_size % 64 == 0.
 *   ep_record_bytes   size of one record.
 *   ep_dest_ranks     dest[t, r] = r if token t has an expert in [r*per_rank, (r+1)*per_rank)
 *                     else -1 (int32 [T, world]); b200_nvfp4_moe_route over it with `world`
 *                     groups gives the rank-major send rows and per-rank counts.
 *   ep_pack_rows      quantises each token row (FP16 / BF16) to NVFP4 once and writes its record
 *                     at every send_pos[t, r] >= 0.
 *   ep_unpack_rows    received records -> packed [rows, H/2], one scale region of
 *                     align128(rows) rows in the block-scaled layout, ids and weights [rows, k]:
 *                     the inputs of b200_nvfp4_fused_moe with rank_ep set. */
B200_NVFP4_API size_t b200_nvfp4_ep_record_bytes(int hidden_size, int num_topk);
B200_NVFP4_API int b200_nvfp4_ep_dest_ranks(const void* topk_ids, void* dest, int num_tokens,
                                            int num_topk, int experts_per_rank, int world,
                                            b200_stream_t stream);
B200_NVFP4_API int b200_nvfp4_ep_pack_rows(void* records, const void* x, const void* topk_ids,
                                           const void* topk_weights, const void* send_pos,
                                           int num_tokens, int hidden_size, int num_topk, int world,
                                           int input_is_bf16, b200_stream_t stream);
B200_NVFP4_API int b200_nvfp4_ep_unpack_rows(void* x_packed, void* x_scale, void* topk_ids,
                                             void* topk_weights, const void* records, int rows,
                                             int hidden_size, int num_topk, b200_stream_t stream);

/* The same hand-off over peer memory instead of a collective: every rank has a receive buffer of
 * `world` slots of `slot_rows` wire records, an int32 count per slot, and a return buffer of `world`
 * slots of `slot_rows` rows, all mapped into the peers' address spaces (peer_*[r] = rank r's buffer
 * as this process addresses it). No counterpart in the reference.
 *   ep_dispatch_p2p   ep_pack_rows, but each record is stored straight into slot `my_rank` of its
 *                     destination rank, the per-destination counts likewise; ret_pos[t, r]
 *                     (int32 [T, world]) receives the row of this rank's return buffer that the
 *                     partial result of token t from rank r will occupy, or -1.
 *   ep_unpack_slots   all world * slot_rows slot rows -> inputs of b200_nvfp4_fused_moe (rank_ep set);
 *                     rows beyond a slot's count get expert id -1 everywhere.
 *   ep_return_p2p     row (s, k) of `partial` [world * slot_rows, row_bytes] -> row (my_rank, k) of
 *                     rank s's return buffer, for k < counts[s].
 * The caller separates dispatch stores / reads and return stores / reads with a barrier over all
 * ranks (the kernels themselves never wait on another GPU). num_tokens <= slot_rows. */
B200_NVFP4_API int b200_nvfp4_ep_dispatch_p2p(const void* const* peer_records,
                                              const void* const* peer_counts, void* ret_pos,
                                              const void* x, const void* topk_ids,
                                              const void* topk_weights, const void* send_pos,
                                              const void* send_counts, const void* send_cu,
                                              int my_rank, int world, int slot_rows, int num_tokens,
                                              int hidden_size, int num_topk, int input_is_bf16,
                                              b200_stream_t stream);
B200_NVFP4_API int b200_nvfp4_ep_unpack_slots(void* x_packed, void* x_scale, void* topk_ids,
                                              void* topk_weights, const void* records,
                                              const void* counts, int world, int slot_rows,
                                              int hidden_size, int num_topk, b200_stream_t stream);
B200_NVFP4_API int b200_nvfp4_ep_return_p2p(const void* const* peer_ret, const void* partial,
                                            const void* counts, int my_rank, int world,
                                            int slot_rows, int row_bytes, b200_stream_t stream);
/* Cross-GPU barrier between the phases of the peer-memory hand-off (no counterpart in the
 * reference, whose hand-off script synchronises through the collective library,
 * benchmarks/integration/benchmark_deepep_handoff.py:466-496). peer_flags[r] points at rank r's
 * `world` int32 flag words (zero before the first call); `epoch` is 1, 2, 3, ... over the calls of
 * one flag set, the same on every rank. The kernel publishes the epoch in flag `my_rank` of every
 * rank (after a system-scope fence) and waits until all of its own flags have reached it. The wait
 * is bounded: after limit_cycles SM clocks (0 = about one second) it stores 9 | (late rank << 8) in
 * the device error word (b200_nvfp4_device_error) and returns; what follows on the stream then
 * runs on incomplete data, which the error word tells. Ranks must be separate GPUs: two launches
 * that wait for each other on one GPU may never run at the same time. */
B200_NVFP4_API int b200_nvfp4_ep_barrier_p2p(const void* const* peer_flags, int my_rank, int world,
                                             int epoch, long long limit_cycles, b200_stream_t stream);

/* ep_reduce_return_p2p over the column window [col_start, col_start + col_count) of the rows only
 * (multiples of 8): with
 * b200_nvfp4_grouped_gemm_columns the down projection can be computed in column blocks and the
 * partial rows of a finished block travel to their sources on a second stream while the next block is
 * computed. No counterpart in the reference. */
B200_NVFP4_API int b200_nvfp4_ep_reduce_return_p2p_columns(const void* const* peer_ret,
                                                           const void* down_output, const void* topk_pos,
                                                           const void* topk_scale, const void* counts,
                                                           int my_rank, int world, int slot_rows,
                                                           int hidden_size, int num_topk, int col_start,
                                                           int col_count, b200_stream_t stream);

/* The same hand-off without a full barrier: per-rank ready words instead (no counterpart in the
 * reference). Every rank keeps 2 * world int32 words in its mapped buffer: word s (s < world) =
 * "source rank s has delivered its records of epoch e", word world + r = "expert rank r has delivered
 * its partial rows of epoch e".
 *   ep_publish_p2p        after the dispatch (slot = 0) or the return stores (slot = world) on the same
 *                         stream: system-scope fence, then `epoch` into word slot + my_rank of every
 *                         peer. Waits for nobody.
 *   ep_unpack_slots_ready ep_unpack_slots whose warps take up the rows of source s once ready[s] has
 *                         reached `epoch`: sources that have delivered are unpacked while others are
 *                         still on their way. ready = this rank's own words [0, world).
 *   ep_sum_p2p            the source's final step - sum of the partial rows that came back, ascending
 *                         rank order, FP32, one rounding (b200_nvfp4_moe_reduce with unit weights over
 *                         ret_pos [num_tokens, world]) - after every ready[r] has reached `epoch`.
 *                         ready = this rank's own words [world, 2 * world).
 * Every wait is bounded by limit_cycles SM clocks (0 = about one second); a word that does not
 * arrive leaves 10 | rank << 8 (records) or 11 | rank << 8 (partial rows) in the device error word,
 * the rows concerned are treated as empty, and the kernel returns. ready = NULL waits for nothing. */
B200_NVFP4_API int b200_nvfp4_ep_publish_p2p(const void* const* peer_flags, int my_rank, int world, int slot,
                                             int epoch, b200_stream_t stream);
B200_NVFP4_API int b200_nvfp4_ep_unpack_slots_ready(void* x_packed, void* x_scale, void* topk_ids,
                                                    void* topk_weights, const void* records,
                                                    const void* counts, int world, int slot_rows,
                                                    int hidden_size, int num_topk, const void* ready,
                                                    int epoch, long long limit_cycles, b200_stream_t stream);
B200_NVFP4_API int b200_nvfp4_ep_sum_p2p(void* output, const void* ret, const void* ret_pos, int num_tokens,
                                         int hidden_size, int world, int out_is_bf16, const void* ready,
                                         int epoch, long long limit_cycles, b200_stream_t stream);

/* ep_return_p2p fused with the reduce step that produces `partial`: the weighted sum over a slot
 * row's local experts (b200_nvfp4_moe_reduce arithmetic, FP16 result, no shared-expert term) is
 * stored straight into the source rank's return slot. down_output / topk_pos / topk_scale are the
 * routed layer's intermediates over all world * slot_rows slot rows. */
B200_NVFP4_API int b200_nvfp4_ep_reduce_return_p2p(const void* const* peer_ret,
                                                   const void* down_output, const void* topk_pos,
                                                   const void* topk_scale, const void* counts,
                                                   int my_rank, int world, int slot_rows,
                                                   int hidden_size, int num_topk,
                                                   b200_stream_t stream);

/* Reads and clears the device word in which a kernel records a timed-out wait (every wait
 * inside the kernels is bounded). SYNCHRONISES the device. *code receives 0 when nothing
 * was recorded. No counterpart in the reference. */
B200_NVFP4_API int b200_nvfp4_device_error(int* code);

/* Forces the tile shape of every GEMM launched afterwards by this process: 64, 128 or 256 =
 * a 128-row tile of that many columns on one CTA; 512 = the 256 x 256 tile on a CTA pair
 * (FP16 output only; FP32 output falls back to 256); 0 restores the built-in choice. For tests and
 * tuning. No counterpart in the reference. Returns B200_NVFP4_INVALID_ARGUMENT for any other
 * value. */
B200_NVFP4_API int b200_nvfp4_set_tile_n(int tile_n);

/* Shape-keyed tile table (no counterpart in the reference's ABI; its RTX 5090 tuning is compiled
 * in). An entry fixes the tile shape - the values of b200_nvfp4_set_tile_n - for exactly one
 * problem: `groups` problems of `rows` x n x k for the dense / batched entry points (grouped = 0),
 * or a grouped call over `groups` groups and `rows` rows in total (grouped = 1); out_f32 selects the
 * FP32-output entry points. tile_n = 0 removes the entry. The built-in rules apply to every problem
 * without an entry; the split-K entry points, the dispatcher's M = 128 / 256 paths and the fused
 * gate/up GEMM never consult the table (their tiles are part of their arithmetic).
 * sm120_nvfp4_b200.ops.autotune_gemm / autotune_grouped_gemm time the candidates on the device
 * and install the fastest. tune_get returns the entry's tile or 0. Thread-safe. */
B200_NVFP4_API int b200_nvfp4_tune_set(int groups, int rows, int n, int k, int out_f32, int grouped,
                                       int tile_n);
B200_NVFP4_API int b200_nvfp4_tune_get(int groups, int rows, int n, int k, int out_f32, int grouped);
B200_NVFP4_API void b200_nvfp4_tune_clear(void);

/* Tile of the most recent GEMM launch of this process (any entry point): the b200_nvfp4_set_tile_n
 * value in the low 16 bits, the number of K ranges reduced inside a cluster (1 = none) above them.
 * For tests of the tile rules and of the table. No counterpart in the reference. */
B200_NVFP4_API int b200_nvfp4_last_launch_tile(void);

/* out_f32[i] = silu(in_f16[i]) = x / (1 + exp(-x)) exactly as b200_nvfp4_moe_act_mul_and_quant and
 * the fused gate/up epilogue evaluate it (the reference's silu(), src/fused_moe/activation.cu:17-19,
 * with this library's fixed-sequence exp): for tests that compare every FP16 input with the CPU
 * oracle. count must be a multiple of 16, both pointers 16-byte aligned. */
B200_NVFP4_API int b200_nvfp4_silu_f16(void* out_f32, const void* in_f16, int count, b200_stream_t stream);

/* Chooses how b200_nvfp4_fused_moe / b200_nvfp4_expert_moe make the down projection's input:
 * enabled != 0 (the default) = b200_nvfp4_grouped_gemm_swiglu_quant, one kernel, gate_up_output
 * is not written; 0 = the reference's two steps (grouped GEMM into gate_up_output, then
 * b200_nvfp4_moe_act_mul_and_quant). Both produce the same bytes. Process-wide. No counterpart in
 * the reference. */
B200_NVFP4_API int b200_nvfp4_set_fused_gate_up(int enabled);

/* Test hook for the bounded waits of the GEMM kernel (no counterpart in the reference). Every
 * mbarrier wait in the kernel gives up after limit_cycles SM clocks (0 restores the default, about
 * one second); a wait that gives up makes its CTA drain, free its tensor memory and store
 * code | (CTA index << 8) in the device error word (codes: 1 operand stage not released, 2 / 5
 * accumulator not handed back, 3 operand stage never ready, 4 tile never finished). With
 * withhold_one_arrival != 0 the NEXT launch (only) leaves out one barrier arrival on purpose - its
 * first k-stage never becomes ready - so that a test can watch a wait run out without anything
 * faulting: that launch returns after the limit, its output is undefined, the error word is set. */
B200_NVFP4_API int b200_nvfp4_set_wait_limit(long long limit_cycles, int withhold_one_arrival);

/* Number of kernel launches this library has issued from the calling process since load
 * (for launch accounting in benchmarks). No counterpart in the reference. */
B200_NVFP4_API long long b200_nvfp4_launch_count(void);

#ifdef __cplusplus
}
#endif

#endif /* B200_NVFP4_H_ */
