// HBM-bound kernels of the fused-MoE path and their C ABI: routing (count -> scan -> stable
// rank), gather to expert-major order, SiLU*up + NVFP4 quantisation, row quantisation and
// the weighted top-k combine. All global accesses on the payload paths are 16-byte vectors.
#include <cstdint>
#include <mutex>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_common.hpp"
#include "internal.hpp"
#include "nvfp4_math.cuh"

namespace b200 {

namespace {

constexpr int kRouteThreads = 1024;
constexpr int kRouteChunk = 1024;   // assignments per routing block (>= max local experts)
constexpr int kMaxExperts = 1024;

// ------------------------------------------------------------------------ routing
//
// Replaces count_local_experts_kernel, build_prefix_and_reset_kernel and the slot
// assignment inside gather_nvfp4_kernel (src/fused_moe/count_and_gather.cu:12-66). The
// reference hands out slots with atomicAdd, so the order inside an expert depends on
// scheduling; here the slot of an assignment is the number of earlier assignments (by flat
// index t * topk + r) to the same expert - deterministic, and one of the orders the
// reference can produce.
//
// Assignments are cut into chunks of 1024 (the last chunk also takes the remainder).
// Pass 1 writes each chunk's per-expert histogram into the first E words of that chunk's
// slice of topk_pos (scratch until pass 3 overwrites it), pass 2 turns the histograms into
// per-chunk bases plus seqlens / cu_seqlens, pass 3 ranks inside each chunk.

__device__ __forceinline__ void chunk_bounds(int chunk, int num_chunks, int total, int& begin, int& end) {
  begin = chunk * kRouteChunk;
  end = (chunk == num_chunks - 1) ? total : begin + kRouteChunk;
}

__global__ void __launch_bounds__(kRouteThreads)
route_count_kernel(const int* __restrict__ topk_ids, int* __restrict__ topk_pos, int total,
                   int num_chunks, int start_expert, int num_expert) {
  __shared__ int hist[kMaxExperts];
  for (int e = threadIdx.x; e < num_expert; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  int begin, end;
  chunk_bounds(blockIdx.x, num_chunks, total, begin, end);
  for (int a = begin + threadIdx.x; a < end; a += blockDim.x) {
    const int e = topk_ids[a] - start_expert;
    if (e >= 0 && e < num_expert) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_expert; e += blockDim.x) topk_pos[begin + e] = hist[e];
}

__global__ void __launch_bounds__(kRouteThreads)
route_scan_kernel(int* __restrict__ topk_pos, int* __restrict__ seqlens,
                  int* __restrict__ cu_seqlens, int num_chunks, int num_expert) {
  __shared__ int warp_sums[32];
  const int e = threadIdx.x;
  int running = 0;
  if (e < num_expert) {
    for (int c0 = 0; c0 < num_chunks; c0 += 8) {
      int v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = (c0 + i < num_chunks) ? topk_pos[(c0 + i) * kRouteChunk + e] : 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (c0 + i < num_chunks) topk_pos[(c0 + i) * kRouteChunk + e] = running;
        running += v[i];
      }
    }
    seqlens[e] = running;
  }
  // exclusive scan over experts -> cu_seqlens
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = (e < num_expert) ? running : 0;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int o = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += o;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sums[lane];
    int wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int o = __shfl_up_sync(0xffffffffu, wi, d);
      if (lane >= d) wi += o;
    }
    warp_sums[lane] = wi - w;
  }
  __syncthreads();
  const int excl = incl - ((e < num_expert) ? running : 0) + warp_sums[warp];
  if (e < num_expert) {
    cu_seqlens[e] = excl;
    if (e == num_expert - 1) cu_seqlens[num_expert] = excl + running;
  }
}

// Ranks the assignments of one chunk in flat-index order. base[e] enters as the first
// grouped row this chunk may use for expert e. Slices of 1024 are processed in order and,
// inside a slice, warps take turns so that ranks follow the flat index.
__device__ __forceinline__ void rank_chunk(const int* __restrict__ topk_ids, int* __restrict__ topk_pos,
                                           int begin, int end, int start_expert, int num_expert,
                                           int* base) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int slice = begin; slice < end; slice += kRouteThreads) {
    const int a = slice + threadIdx.x;
    int e = -1;
    if (a < end) {
      e = topk_ids[a] - start_expert;
      if (e < 0 || e >= num_expert) e = -1;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int before = __popc(peers & ((1u << lane) - 1u));
    const int count = __popc(peers);
    int pos = -1;
    for (int w = 0; w < kRouteThreads / 32; ++w) {
      if (warp == w && e >= 0) {
        pos = base[e] + before;
      }
      __syncwarp();
      if (warp == w && e >= 0 && before == 0) base[e] += count;
      __syncthreads();
    }
    if (a < end) topk_pos[a] = pos;
  }
}

__global__ void __launch_bounds__(kRouteThreads)
route_rank_kernel(const int* __restrict__ topk_ids, int* __restrict__ topk_pos,
                  const int* __restrict__ cu_seqlens, int total, int num_chunks, int start_expert,
                  int num_expert) {
  __shared__ int base[kMaxExperts];
  int begin, end;
  chunk_bounds(blockIdx.x, num_chunks, total, begin, end);
  for (int e = threadIdx.x; e < num_expert; e += blockDim.x) base[e] = topk_pos[begin + e] + cu_seqlens[e];
  __syncthreads();
  rank_chunk(topk_ids, topk_pos, begin, end, start_expert, num_expert, base);
}

// Whole routing in one block, for fewer than 2048 assignments (no scratch needed).
__global__ void __launch_bounds__(kRouteThreads)
route_small_kernel(const int* __restrict__ topk_ids, int* __restrict__ topk_pos,
                   int* __restrict__ seqlens, int* __restrict__ cu_seqlens, int total,
                   int start_expert, int num_expert) {
  __shared__ int base[kMaxExperts + 1];
  __shared__ int count[kMaxExperts];
  for (int e = threadIdx.x; e < num_expert; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int a = threadIdx.x; a < total; a += blockDim.x) {
    const int e = topk_ids[a] - start_expert;
    if (e >= 0 && e < num_expert) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < num_expert; ++e) {
      base[e] = run;
      run += count[e];
    }
    base[num_expert] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= num_expert; e += blockDim.x) {
    cu_seqlens[e] = base[e];
    if (e < num_expert) seqlens[e] = count[e];
  }
  __syncthreads();
  rank_chunk(topk_ids, topk_pos, 0, total, start_expert, num_expert, base);
}

// ------------------------------------------------------------------------- gather
//
// Replaces the copy part of gather_nvfp4_kernel (count_and_gather.cu:66-91): one warp per
// assignment copies the packed row with 16-byte vectors and re-addresses the row's scale
// bytes from the token's region to the expert's region, one 4-byte atom row at a time.
__global__ void __launch_bounds__(256)
gather_kernel(uint8_t* __restrict__ grouped_input, uint8_t* __restrict__ grouped_scale,
              const uint8_t* __restrict__ input, const uint8_t* __restrict__ input_scale,
              const int* __restrict__ topk_ids, const int* __restrict__ topk_pos,
              const int* __restrict__ cu_seqlens, int total, int hidden, int num_topk,
              int start_expert, long long group_scale_stride) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int row_bytes = hidden >> 1;
  const int nkb = (hidden + 15) >> 4;
  const int kt = (nkb + 3) >> 2;
  for (int a = blockIdx.x * warps_per_block + (threadIdx.x >> 5); a < total;
       a += gridDim.x * warps_per_block) {
    const int grouped_row = topk_pos[a];
    if (grouped_row < 0) continue;
    const int expert = topk_ids[a] - start_expert;
    const int position = grouped_row - cu_seqlens[expert];
    const int token = a / num_topk;
    const uint4* src = reinterpret_cast<const uint4*>(input + static_cast<long long>(token) * row_bytes);
    uint4* dst = reinterpret_cast<uint4*>(grouped_input + static_cast<long long>(grouped_row) * row_bytes);
    // eight 16-byte vectors (and four scale words) per lane are loaded before the first is stored
    const int vecs = row_bytes >> 4;
    for (int base = lane; base < vecs; base += 256) {
      uint4 buf[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (base + 32 * u < vecs) buf[u] = src[base + 32 * u];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (base + 32 * u < vecs) dst[base + 32 * u] = buf[u];
    }
    const uint8_t* s_row = input_scale + sf_offset(token, 0, kt);
    uint8_t* d_row = grouped_scale + expert * group_scale_stride + sf_offset(position, 0, kt);
    for (int base = lane; base < kt; base += 128) {
      uint32_t v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = base + 32 * u;
        if (j < kt) {
          v[u] = *reinterpret_cast<const uint32_t*>(s_row + static_cast<long long>(j) * 512);
          const int valid = nkb - 4 * j;
          if (valid < 4) v[u] &= (1u << (8 * valid)) - 1u;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = base + 32 * u;
        if (j < kt) *reinterpret_cast<uint32_t*>(d_row + static_cast<long long>(j) * 512) = v[u];
      }
    }
  }
}

// ------------------------------------------------------------ quantising kernels
//
// Work item = 16 consecutive values of one live row; a warp covers 32 consecutive blocks of
// a row (512 values). Only rows below cu_seqlens[E] are visited, never the padded
// E * m_pad space the reference grid-strides over (activation.cu:182-188).

struct RowMap {
  int expert;
  int row;  // row inside the expert, or -1 when the grouped row belongs to no expert
};

__device__ __forceinline__ RowMap map_row(const int* s_cu, const int* seqlens, int num_expert, int grouped_row) {
  int lo = 0, hi = num_expert;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (s_cu[mid] <= grouped_row) lo = mid; else hi = mid;
  }
  RowMap m;
  m.expert = lo;
  m.row = grouped_row - s_cu[lo];
  if (m.row >= seqlens[lo]) m.row = -1;
  return m;
}

__device__ __forceinline__ void load16(const __half* p, float (&v)[16]) {
  const uint4 a = reinterpret_cast<const uint4*>(p)[0];
  const uint4 b = reinterpret_cast<const uint4*>(p)[1];
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
    v[2 * i] = __low2float(h);
    v[2 * i + 1] = __high2float(h);
  }
}

__device__ __forceinline__ void load16(const __nv_bfloat16* p, float (&v)[16]) {
  const uint4 a = reinterpret_cast<const uint4*>(p)[0];
  const uint4 b = reinterpret_cast<const uint4*>(p)[1];
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// kMode 0: silu(gate) * up from FP16 [rows, 2*width]; 1: FP16 rows; 2: BF16 rows; 3: FP32 rows.
template <int kMode>
__global__ void __launch_bounds__(256)
quant_rows_kernel(uint8_t* __restrict__ output, uint8_t* __restrict__ output_scale,
                  const void* __restrict__ input, const int* __restrict__ seqlens,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ row_map, int num_expert,
                  int width, long long group_scale_stride) {
  extern __shared__ int s_cu[];
  for (int e = threadIdx.x; e <= num_expert; e += blockDim.x) s_cu[e] = cu_seqlens[e];
  __syncthreads();
  const int total_rows = s_cu[num_expert];
  const int lane = threadIdx.x & 31;
  const int nkb = width >> 4;
  const int kt = (nkb + 3) >> 2;
  const int groups_per_row = (nkb + 31) >> 5;
  const long long items = static_cast<long long>(total_rows) * groups_per_row;
  const int warps_per_block = blockDim.x >> 5;
  for (long long item = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
       item < items; item += static_cast<long long>(gridDim.x) * warps_per_block) {
    const int grouped_row = static_cast<int>(item / groups_per_row);
    const int kb = static_cast<int>(item % groups_per_row) * 32 + lane;
    const RowMap m = map_row(s_cu, seqlens, num_expert, grouped_row);
    const bool live = m.row >= 0 && kb < nkb;
    uint8_t code = 0;
    if (live) {
      float v[16];
      // optional gather: grouped row r is read from input row row_map[r]
      const long long in_row = row_map ? static_cast<long long>(row_map[grouped_row]) : grouped_row;
      if constexpr (kMode == 0) {
        const __half* gate = static_cast<const __half*>(input) + in_row * width * 2 + kb * 16;
        float g[16], u[16];
        load16(gate, g);
        load16(gate + width, u);
        silu_mul_block16(g, u, v);
      } else if constexpr (kMode == 1) {
        load16(static_cast<const __half*>(input) + in_row * width + kb * 16, v);
      } else if constexpr (kMode == 2) {
        load16(static_cast<const __nv_bfloat16*>(input) + in_row * width + kb * 16, v);
      } else {
        const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(input) + in_row * width + kb * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 f = src[i];
          v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
      }
      uint32_t lo, hi;
      code = quantize_block16(v, lo, hi);
      *reinterpret_cast<uint2*>(output + static_cast<long long>(grouped_row) * (width >> 1) + kb * 8) =
          make_uint2(lo, hi);
    }
    // four neighbouring lanes own the four bytes of one atom row: merge and store once
    uint32_t word = static_cast<uint32_t>(code) << (8 * (lane & 3));
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);
    if ((lane & 3) == 0 && m.row >= 0 && kb < nkb) {
      *reinterpret_cast<uint32_t*>(output_scale + m.expert * group_scale_stride +
                                   sf_offset(m.row, kb, kt)) = word;
    }
  }
}

// ------------------------------------------------------------------------- reduce
//
// Replaces reduce_nvfp4_kernel (src/fused_moe/reduce.cu:12-35): one thread per 8 output
// columns, FP32 accumulation in route order starting from the shared-expert row, one
// rounding at the end.
template <bool kOutBf16>
__global__ void __launch_bounds__(256)
reduce_kernel(void* __restrict__ output, const __half* __restrict__ down_output,
              const int* __restrict__ topk_pos, const float* __restrict__ topk_scale,
              const __half* __restrict__ shared_output, int num_tokens, int hidden, int num_topk) {
  const int chunks = hidden >> 3;
  const long long items = static_cast<long long>(num_tokens) * chunks;
  for (long long item = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; item < items;
       item += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int token = static_cast<int>(item / chunks);
    const int col = static_cast<int>(item % chunks) * 8;
    float acc[8];
    if (shared_output) {
      const uint4 s = *reinterpret_cast<const uint4*>(shared_output + static_cast<long long>(token) * hidden + col);
      const uint32_t w[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
        acc[2 * i] = __low2float(h);
        acc[2 * i + 1] = __high2float(h);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
    }
    const int* pos = topk_pos + static_cast<long long>(token) * num_topk;
    const float* wts = topk_scale + static_cast<long long>(token) * num_topk;
    for (int r = 0; r < num_topk; ++r) {
      const int row = pos[r];
      if (row < 0) continue;
      const float wt = wts[r];
      const uint4 d = *reinterpret_cast<const uint4*>(down_output + static_cast<long long>(row) * hidden + col);
      const uint32_t w[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
        acc[2 * i] = __fmaf_rn(__low2float(h), wt, acc[2 * i]);
        acc[2 * i + 1] = __fmaf_rn(__high2float(h), wt, acc[2 * i + 1]);
      }
    }
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (kOutBf16) {
        const __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        ow[i] = *reinterpret_cast<const uint32_t*>(&b);
      } else {
        const __half2 h = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
        ow[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
    if constexpr (kOutBf16) {
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(output) + static_cast<long long>(token) * hidden + col) = o;
    } else {
      *reinterpret_cast<uint4*>(static_cast<__half*>(output) + static_cast<long long>(token) * hidden + col) = o;
    }
  }
}

// ------------------------------------------------------------------------- router
//
// Router step in front of the routed layer: score = sigmoid(logit), the num_topk largest per
// token (ties to the lower expert id), weight = score / sum of the selected scores (sum in
// selection order). The reference library leaves this step to its caller. One warp per token:
// the scores sit in shared memory, every round each lane scans its strided share and the warp
// agrees on the best (score, lowest id) with shuffles.
__global__ void __launch_bounds__(256)
router_topk_kernel(const float* __restrict__ logits, int* __restrict__ topk_ids,
                   float* __restrict__ topk_weights, int num_tokens, int num_experts, int num_topk) {
  extern __shared__ float s_scores[];
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  float* score = s_scores + static_cast<size_t>(threadIdx.x >> 5) * num_experts;
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < num_tokens; t += gridDim.x * warps_per_block) {
    const float* row = logits + static_cast<long long>(t) * num_experts;
    for (int e = lane; e < num_experts; e += 32)
      score[e] = __fdiv_rn(1.0f, __fadd_rn(1.0f, nvfp4_expf(-row[e])));
    __syncwarp();
    float sum = 0.0f;
    float my_weight = 0.0f;   // lane r keeps the score of rank r (num_topk <= 32 per pass)
    int my_id = -1;
    for (int r = 0; r < num_topk; ++r) {
      float best = -1.0f;
      int best_id = 0x7fffffff;
      for (int e = lane; e < num_experts; e += 32) {
        const float v = score[e];
        if (v > best) { best = v; best_id = e; }   // ascending e: the first maximum has the lowest id
      }
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, d);
        const int oi = __shfl_xor_sync(0xffffffffu, best_id, d);
        if (ov > best || (ov == best && oi < best_id)) { best = ov; best_id = oi; }
      }
      const bool found = best >= 0.0f;
      if (found) {
        sum = r == 0 ? best : __fadd_rn(sum, best);
        if (lane == 0) score[best_id] = -1.0f;
      }
      if ((r & 31) == lane) { my_weight = found ? best : 0.0f; my_id = found ? best_id : -1; }
      __syncwarp();
      if ((r & 31) == 31 || r == num_topk - 1) {
        // flush up to 32 selections; the divisor needs the complete sum, so weights are
        // normalised in a second pass below
        const int base = r & ~31;
        if (base + lane <= r) {
          topk_ids[static_cast<long long>(t) * num_topk + base + lane] = my_id;
          topk_weights[static_cast<long long>(t) * num_topk + base + lane] = my_weight;
        }
      }
    }
    __syncwarp();
    for (int r = lane; r < num_topk; r += 32) {
      float* w = topk_weights + static_cast<long long>(t) * num_topk + r;
      *w = __fdiv_rn(*w, sum);
    }
    __syncwarp();
  }
}

__global__ void __launch_bounds__(256)
move_rows_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src,
                 const int* __restrict__ index, int count, int fanout, int row_bytes, bool scatter) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int vecs = row_bytes >> 4;
  for (int i = blockIdx.x * warps_per_block + (threadIdx.x >> 5); i < count; i += gridDim.x * warps_per_block) {
    const int idx = index[i];
    if (idx < 0) continue;
    const long long src_row = scatter ? i / fanout : idx;
    const long long dst_row = scatter ? idx : i;
    const uint4* s4 = reinterpret_cast<const uint4*>(src + src_row * row_bytes);
    uint4* d4 = reinterpret_cast<uint4*>(dst + dst_row * row_bytes);
    for (int v = lane; v < vecs; v += 32) d4[v] = s4[v];
  }
}

// out[i] = silu(in[i]) for FP16 inputs, sixteen per thread through silu_mul_block16 (up = 1): the
// activation exactly as the quantising kernels and the fused GEMM epilogue evaluate it, exposed so
// that a test can compare every FP16 input with the oracle.
__global__ void __launch_bounds__(256)
silu_f16_kernel(float* __restrict__ out, const __half* __restrict__ in, int blocks16) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= blocks16) return;
  float g[16], u[16], v[16];
  load16(in + static_cast<long long>(b) * 16, g);
#pragma unroll
  for (int i = 0; i < 16; ++i) u[i] = 1.0f;
  silu_mul_block16(g, u, v);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    reinterpret_cast<float4*>(out + static_cast<long long>(b) * 16)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

int moe_count_and_gather(void* gate_up_input, void* gate_up_input_scale, const void* input,
                         const void* input_scale, const void* topk_ids, void* topk_pos,
                         void* seqlens, void* cu_seqlens, int num_tokens, int hidden_size,
                         int num_topk, int num_expert_local, int rank_ep, int input_scale_m_pad,
                         int grouped_scale_m_pad, bool zero_scales, cudaStream_t stream) {
  const long long total64 = static_cast<long long>(num_tokens) * num_topk;
  if (gate_up_input == nullptr || gate_up_input_scale == nullptr || input == nullptr ||
      input_scale == nullptr || topk_ids == nullptr || topk_pos == nullptr || seqlens == nullptr ||
      cu_seqlens == nullptr || num_tokens <= 0 || num_topk <= 0 || hidden_size <= 0 ||
      (hidden_size % 32) != 0 || num_expert_local <= 0 || num_expert_local > kMaxExperts ||
      rank_ep < 0 || total64 > 0x7fffffffLL || input_scale_m_pad < num_tokens ||
      (grouped_scale_m_pad % 128) != 0 || grouped_scale_m_pad < 128 || !aligned16(input) ||
      !aligned16(gate_up_input) || !aligned16(input_scale) || !aligned16(gate_up_input_scale)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  const DeviceInfo& dev = current_device_info();
  if (!dev.ok) return B200_NVFP4_CUDA_ERROR;
  const int total = static_cast<int>(total64);
  const int start_expert = rank_ep * num_expert_local;
  const long long group_stride = static_cast<long long>(grouped_scale_m_pad) * scale_k_padded(hidden_size);
  if (zero_scales) {
    if (cudaMemsetAsync(gate_up_input_scale, 0, static_cast<size_t>(num_expert_local) * group_stride,
                        stream) != cudaSuccess)
      return B200_NVFP4_CUDA_ERROR;
  }
  const int* ids = static_cast<const int*>(topk_ids);
  int* pos = static_cast<int*>(topk_pos);
  int* sl = static_cast<int*>(seqlens);
  int* cu = static_cast<int*>(cu_seqlens);
  const int num_chunks = total / kRouteChunk;
  if (num_chunks <= 1) {
    route_small_kernel<<<1, kRouteThreads, 0, stream>>>(ids, pos, sl, cu, total, start_expert,
                                                        num_expert_local);
    count_launch();
  } else {
    route_count_kernel<<<num_chunks, kRouteThreads, 0, stream>>>(ids, pos, total, num_chunks,
                                                                 start_expert, num_expert_local);
    route_scan_kernel<<<1, kRouteThreads, 0, stream>>>(pos, sl, cu, num_chunks, num_expert_local);
    route_rank_kernel<<<num_chunks, kRouteThreads, 0, stream>>>(ids, pos, cu, total, num_chunks,
                                                                start_expert, num_expert_local);
    count_launch(3);
  }
  if (launch_status() != B200_NVFP4_SUCCESS) return B200_NVFP4_CUDA_ERROR;
  int blocks = (total + 7) / 8;
  const int max_blocks = dev.sm_count * 8;
  if (blocks > max_blocks) blocks = max_blocks;
  gather_kernel<<<blocks, 256, 0, stream>>>(
      static_cast<uint8_t*>(gate_up_input), static_cast<uint8_t*>(gate_up_input_scale),
      static_cast<const uint8_t*>(input), static_cast<const uint8_t*>(input_scale), ids, pos, cu,
      total, hidden_size, num_topk, start_expert, group_stride);
  count_launch();
  return launch_status();
}

template <int kMode>
int launch_quant(void* output, void* output_scale, const void* input, const void* seqlens,
                 const void* cu_seqlens, const void* row_map, int num_expert_local, int total_rows,
                 int width, int grouped_scale_m_pad, bool zero_scales, cudaStream_t stream) {
  if (output == nullptr || output_scale == nullptr || input == nullptr || seqlens == nullptr ||
      cu_seqlens == nullptr || num_expert_local <= 0 || num_expert_local > kMaxExperts ||
      width <= 0 || (width % 32) != 0 || grouped_scale_m_pad < 128 ||
      (grouped_scale_m_pad % 128) != 0 || !aligned16(output) || !aligned16(input) ||
      !aligned16(output_scale)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  const DeviceInfo& dev = current_device_info();
  if (!dev.ok) return B200_NVFP4_CUDA_ERROR;
  const long long group_stride = static_cast<long long>(grouped_scale_m_pad) * scale_k_padded(width);
  if (zero_scales) {
    if (cudaMemsetAsync(output_scale, 0, static_cast<size_t>(num_expert_local) * group_stride,
                        stream) != cudaSuccess)
      return B200_NVFP4_CUDA_ERROR;
  }
  // total_rows is only an upper bound for the grid; the kernel reads the live row count
  // from cu_seqlens[E] on the device.
  const long long groups_per_row = ((width >> 4) + 31) >> 5;
  const long long max_blocks = static_cast<long long>(dev.sm_count) * 8;
  long long blocks = max_blocks;  // total_rows <= 0: row count unknown on the host
  if (total_rows > 0) blocks = (static_cast<long long>(total_rows) * groups_per_row + 7) / 8;
  if (blocks > max_blocks) blocks = max_blocks;
  if (blocks < 1) blocks = 1;
  quant_rows_kernel<kMode><<<static_cast<int>(blocks), 256, (num_expert_local + 1) * sizeof(int), stream>>>(
      static_cast<uint8_t*>(output), static_cast<uint8_t*>(output_scale), input,
      static_cast<const int*>(seqlens), static_cast<const int*>(cu_seqlens),
      static_cast<const int*>(row_map), num_expert_local, width, group_stride);
  count_launch();
  return launch_status();
}

int moe_act_mul_and_quant(void* output, void* output_scale, const void* gate_up, const void* seqlens,
                          const void* cu_seqlens, int num_expert_local, int total_rows,
                          int grouped_scale_m_pad, int intermediate_size, bool zero_scales,
                          cudaStream_t stream) {
  return launch_quant<0>(output, output_scale, gate_up, seqlens, cu_seqlens, nullptr, num_expert_local,
                         total_rows, intermediate_size, grouped_scale_m_pad, zero_scales, stream);
}

int moe_quantize_expert(void* output, void* output_scale, const void* input, const void* seqlens,
                        const void* cu_seqlens, const void* row_map, int num_expert_local,
                        int total_rows, int hidden_size, int grouped_scale_m_pad, int input_dtype,
                        bool zero_scales, cudaStream_t stream) {
  switch (input_dtype) {   // 0 FP16, 1 BF16, 2 FP32
    case 0:
      return launch_quant<1>(output, output_scale, input, seqlens, cu_seqlens, row_map, num_expert_local,
                             total_rows, hidden_size, grouped_scale_m_pad, zero_scales, stream);
    case 1:
      return launch_quant<2>(output, output_scale, input, seqlens, cu_seqlens, row_map, num_expert_local,
                             total_rows, hidden_size, grouped_scale_m_pad, zero_scales, stream);
    case 2:
      return launch_quant<3>(output, output_scale, input, seqlens, cu_seqlens, row_map, num_expert_local,
                             total_rows, hidden_size, grouped_scale_m_pad, zero_scales, stream);
    default:
      return B200_NVFP4_INVALID_ARGUMENT;
  }
}

// Routing only (no payload movement): seqlens / cu_seqlens / topk_pos as in
// moe_count_and_gather.
int moe_route(const void* topk_ids, void* topk_pos, void* seqlens, void* cu_seqlens, int num_tokens,
              int num_topk, int num_expert_local, int rank_ep, cudaStream_t stream) {
  const long long total64 = static_cast<long long>(num_tokens) * num_topk;
  if (topk_ids == nullptr || topk_pos == nullptr || seqlens == nullptr || cu_seqlens == nullptr ||
      num_tokens <= 0 || num_topk <= 0 || num_expert_local <= 0 || num_expert_local > kMaxExperts ||
      rank_ep < 0 || total64 > 0x7fffffffLL) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  const int total = static_cast<int>(total64);
  const int start_expert = rank_ep * num_expert_local;
  const int* ids = static_cast<const int*>(topk_ids);
  int* pos = static_cast<int*>(topk_pos);
  int* sl = static_cast<int*>(seqlens);
  int* cu = static_cast<int*>(cu_seqlens);
  const int num_chunks = total / kRouteChunk;
  if (num_chunks <= 1) {
    route_small_kernel<<<1, kRouteThreads, 0, stream>>>(ids, pos, sl, cu, total, start_expert,
                                                        num_expert_local);
    count_launch();
  } else {
    route_count_kernel<<<num_chunks, kRouteThreads, 0, stream>>>(ids, pos, total, num_chunks,
                                                                 start_expert, num_expert_local);
    route_scan_kernel<<<1, kRouteThreads, 0, stream>>>(pos, sl, cu, num_chunks, num_expert_local);
    route_rank_kernel<<<num_chunks, kRouteThreads, 0, stream>>>(ids, pos, cu, total, num_chunks,
                                                                start_expert, num_expert_local);
    count_launch(3);
  }
  return launch_status();
}

// Row movers of the expert-parallel driver (16-byte vectors, one warp per row).
//   scatter: dst[pos[a]] = src[a / fanout]   for every a < count with pos[a] >= 0
//   gather:  dst[i]      = src[map[i]]       for every i < count with map[i] >= 0
int moe_move_rows(void* dst, const void* src, const void* index, int count, int fanout, int row_bytes,
                  bool scatter, cudaStream_t stream) {
  if (dst == nullptr || src == nullptr || index == nullptr || count <= 0 || fanout <= 0 ||
      row_bytes <= 0 || (row_bytes % 16) != 0 || !aligned16(dst) || !aligned16(src)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  const DeviceInfo& dev = current_device_info();
  if (!dev.ok) return B200_NVFP4_CUDA_ERROR;
  int blocks = (count + 7) / 8;
  const int max_blocks = dev.sm_count * 8;
  if (blocks > max_blocks) blocks = max_blocks;
  move_rows_kernel<<<blocks, 256, 0, stream>>>(static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src),
                                               static_cast<const int*>(index), count, fanout, row_bytes,
                                               scatter);
  count_launch();
  return launch_status();
}

int moe_router_topk(const void* logits, void* topk_ids, void* topk_weights, int num_tokens,
                    int num_experts, int num_topk, cudaStream_t stream) {
  if (logits == nullptr || topk_ids == nullptr || topk_weights == nullptr || num_tokens <= 0 ||
      num_experts <= 0 || num_experts > 4096 || num_topk <= 0 || num_topk > num_experts) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  const DeviceInfo& dev = current_device_info();
  if (!dev.ok) return B200_NVFP4_CUDA_ERROR;
  // eight warps per block keep one score row each in shared memory: 128 KiB at the 4096-expert
  // limit, which needs the opt-in above the 48 KiB default (once per device)
  constexpr size_t kMaxRouterSmem = static_cast<size_t>(8) * 4096 * sizeof(float);
  static std::once_flag once[64];
  static cudaError_t attr_status[64];
  if (dev.device < 0 || dev.device >= 64) return B200_NVFP4_CUDA_ERROR;
  std::call_once(once[dev.device], [&] {
    attr_status[dev.device] = cudaFuncSetAttribute(router_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   static_cast<int>(kMaxRouterSmem));
  });
  if (attr_status[dev.device] != cudaSuccess) return B200_NVFP4_CUDA_ERROR;
  int blocks = (num_tokens + 7) / 8;
  const int max_blocks = dev.sm_count * 8;
  if (blocks > max_blocks) blocks = max_blocks;
  router_topk_kernel<<<blocks, 256, static_cast<size_t>(8) * num_experts * sizeof(float), stream>>>(
      static_cast<const float*>(logits), static_cast<int*>(topk_ids), static_cast<float*>(topk_weights),
      num_tokens, num_experts, num_topk);
  count_launch();
  return launch_status();
}

int moe_silu_f16(void* out_f32, const void* in_f16, int count, cudaStream_t stream) {
  if (out_f32 == nullptr || in_f16 == nullptr || count <= 0 || (count % 16) != 0 || !aligned16(out_f32) ||
      !aligned16(in_f16)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  const int blocks16 = count / 16;
  silu_f16_kernel<<<(blocks16 + 255) / 256, 256, 0, stream>>>(static_cast<float*>(out_f32),
                                                             static_cast<const __half*>(in_f16), blocks16);
  count_launch();
  return launch_status();
}

int moe_reduce(void* output, const void* down_output, const void* topk_pos, const void* topk_scale,
               const void* shared_output, int num_tokens, int hidden_size, int num_topk,
               bool out_is_bf16, cudaStream_t stream) {
  if (output == nullptr || down_output == nullptr || topk_pos == nullptr || topk_scale == nullptr ||
      num_tokens <= 0 || hidden_size <= 0 || (hidden_size % 8) != 0 || num_topk <= 0 ||
      !aligned16(output) || !aligned16(down_output) || !aligned16(shared_output)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  const DeviceInfo& dev = current_device_info();
  if (!dev.ok) return B200_NVFP4_CUDA_ERROR;
  const long long items = static_cast<long long>(num_tokens) * (hidden_size >> 3);
  long long blocks = (items + 255) / 256;
  const long long max_blocks = static_cast<long long>(dev.sm_count) * 16;
  if (blocks > max_blocks) blocks = max_blocks;
  if (out_is_bf16) {
    reduce_kernel<true><<<static_cast<int>(blocks), 256, 0, stream>>>(
        output, static_cast<const __half*>(down_output), static_cast<const int*>(topk_pos),
        static_cast<const float*>(topk_scale), static_cast<const __half*>(shared_output), num_tokens,
        hidden_size, num_topk);
  } else {
    reduce_kernel<false><<<static_cast<int>(blocks), 256, 0, stream>>>(
        output, static_cast<const __half*>(down_output), static_cast<const int*>(topk_pos),
        static_cast<const float*>(topk_scale), static_cast<const __half*>(shared_output), num_tokens,
        hidden_size, num_topk);
  }
  count_launch();
  return launch_status();
}

}  // namespace b200
