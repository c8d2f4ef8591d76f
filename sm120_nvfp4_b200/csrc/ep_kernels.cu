// Kernels of the expert-parallel hand-off: what a rank sends to the ranks that own a token's
// experts, and how the receiving rank turns it back into the inputs of the fused MoE.
//
// The reference's 2-GPU hand-off script (benchmarks/integration/benchmark_deepep_handoff.py:
// 356-364) ships one BF16 row per (token, expert) assignment. Here a token is shipped ONCE to
// each rank that owns at least one of its experts, already quantised to NVFP4 (the quantiser
// works on one row at a time, so quantising before or after the exchange gives the same
// bytes), together with its expert ids and route weights. One wire record is
//
//     [ payload  H/2 bytes | scales H/16 bytes (k-block order) | ids k x int32 | weights k x f32 ]
//
// padded to a multiple of 16 bytes: 4096 bytes for H = 7168, k = 8, against 8 x 14336 bytes
// of BF16 rows. The receiver unpacks records into the packed activation matrix, the 512-byte
// atom scale layout, and the id / weight arrays that b200_nvfp4_fused_moe takes with
// rank_ep set, which filters each token's experts to the local interval.
#include <cstdint>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "b200_nvfp4.h"
#include "host_common.hpp"
#include "internal.hpp"
#include "nvfp4_math.cuh"

namespace b200 {
namespace {

constexpr int kMaxWorld = 64;

__host__ __device__ inline long long record_bytes(int hidden, int num_topk) {
  const long long raw = hidden / 2 + hidden / 16 + 8LL * num_topk;
  return (raw + 15) / 16 * 16;
}

// dest[t, r] = r when token t has an expert in [r * per_rank, (r + 1) * per_rank), else -1.
// Routing this array with the ordinary route kernels (W "experts") yields, per token and
// rank, the row of the send buffer (rank-major, token order inside a rank) or -1.
__global__ void __launch_bounds__(256)
ep_dest_kernel(const int* __restrict__ topk_ids, int* __restrict__ dest, int num_tokens, int num_topk,
               int per_rank, int world) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= num_tokens) return;
  unsigned long long mask = 0ull;
  for (int j = 0; j < num_topk; ++j) {
    const int id = topk_ids[static_cast<long long>(t) * num_topk + j];
    if (id >= 0) {
      const int r = id / per_rank;
      if (r < world) mask |= 1ull << r;
    }
  }
  for (int r = 0; r < world; ++r) dest[static_cast<long long>(t) * world + r] = ((mask >> r) & 1ull) ? r : -1;
}

__device__ __forceinline__ void load16_bf16(const __nv_bfloat16* p, float (&v)[16]) {
  const uint4 a = reinterpret_cast<const uint4*>(p)[0];
  const uint4 b = reinterpret_cast<const uint4*>(p)[1];
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ void load16_f16(const __half* p, float (&v)[16]) {
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

// One warp per (token, group of 512 values): each lane quantises 16 values once and stores
// the 8 payload bytes into every record of the token; four lanes merge their scale bytes into
// one 32-bit store. The first warp of a token also writes ids and weights.
template <bool kBf16>
__global__ void __launch_bounds__(256)
ep_pack_kernel(uint8_t* __restrict__ records, const void* __restrict__ x, const int* __restrict__ topk_ids,
               const float* __restrict__ topk_weights, const int* __restrict__ pos, int num_tokens,
               int hidden, int num_topk, int world) {
  const int lane = threadIdx.x & 31;
  const int nkb = hidden >> 4;
  const int groups_per_row = (nkb + 31) >> 5;
  const long long rb = record_bytes(hidden, num_topk);
  const int payload_bytes = hidden >> 1;
  const long long items = static_cast<long long>(num_tokens) * groups_per_row;
  const int warps_per_block = blockDim.x >> 5;
  for (long long item = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
       item < items; item += static_cast<long long>(gridDim.x) * warps_per_block) {
    const int t = static_cast<int>(item / groups_per_row);
    const int group = static_cast<int>(item % groups_per_row);
    const int kb = group * 32 + lane;
    const bool live = kb < nkb;
    uint32_t lo = 0, hi = 0;
    uint8_t code = 0;
    if (live) {
      float v[16];
      if constexpr (kBf16) {
        load16_bf16(static_cast<const __nv_bfloat16*>(x) + static_cast<long long>(t) * hidden + kb * 16, v);
      } else {
        load16_f16(static_cast<const __half*>(x) + static_cast<long long>(t) * hidden + kb * 16, v);
      }
      code = quantize_block16(v, lo, hi);
    }
    uint32_t word = static_cast<uint32_t>(code) << (8 * (lane & 3));
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);
    for (int r = 0; r < world; ++r) {
      const int row = pos[static_cast<long long>(t) * world + r];
      if (row < 0) continue;
      uint8_t* rec = records + static_cast<long long>(row) * rb;
      if (live) {
        *reinterpret_cast<uint2*>(rec + kb * 8) = make_uint2(lo, hi);
        if ((lane & 3) == 0) *reinterpret_cast<uint32_t*>(rec + payload_bytes + kb) = word;
      }
      if (group == 0) {
        int* rid = reinterpret_cast<int*>(rec + payload_bytes + nkb);
        float* rw = reinterpret_cast<float*>(rec + payload_bytes + nkb + 4 * num_topk);
        for (int j = lane; j < num_topk; j += 32) {
          rid[j] = topk_ids[static_cast<long long>(t) * num_topk + j];
          rw[j] = topk_weights[static_cast<long long>(t) * num_topk + j];
        }
      }
    }
  }
}

// One warp per received record: payload with 16-byte vectors, scale words into the atom layout
// of a single region (row = received row), ids and weights into their arrays.
__global__ void __launch_bounds__(256)
ep_unpack_kernel(uint8_t* __restrict__ x_packed, uint8_t* __restrict__ x_scale, int* __restrict__ ids,
                 float* __restrict__ weights, const uint8_t* __restrict__ records, int rows, int hidden,
                 int num_topk) {
  const int lane = threadIdx.x & 31;
  const int nkb = hidden >> 4;
  const int kt = (nkb + 3) >> 2;
  const long long rb = record_bytes(hidden, num_topk);
  const int payload_bytes = hidden >> 1;
  const int warps_per_block = blockDim.x >> 5;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += gridDim.x * warps_per_block) {
    const uint8_t* rec = records + static_cast<long long>(row) * rb;
    const uint4* src = reinterpret_cast<const uint4*>(rec);
    uint4* dst = reinterpret_cast<uint4*>(x_packed + static_cast<long long>(row) * payload_bytes);
    for (int i = lane; i < (payload_bytes >> 4); i += 32) dst[i] = src[i];
    uint8_t* s_row = x_scale + sf_offset(row, 0, kt);
    for (int j = lane; j < kt; j += 32) {
      uint32_t v;
      const int valid = nkb - 4 * j;
      if (valid >= 4) {
        v = *reinterpret_cast<const uint32_t*>(rec + payload_bytes + 4 * j);
      } else {
        v = 0;
        for (int b = 0; b < valid; ++b) v |= static_cast<uint32_t>(rec[payload_bytes + 4 * j + b]) << (8 * b);
      }
      *reinterpret_cast<uint32_t*>(s_row + static_cast<long long>(j) * 512) = v;
    }
    const int* rid = reinterpret_cast<const int*>(rec + payload_bytes + nkb);
    const float* rw = reinterpret_cast<const float*>(rec + payload_bytes + nkb + 4 * num_topk);
    for (int j = lane; j < num_topk; j += 32) {
      ids[static_cast<long long>(row) * num_topk + j] = rid[j];
      weights[static_cast<long long>(row) * num_topk + j] = rw[j];
    }
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_launch() {
  return cudaPeekAtLastError() == cudaSuccess ? B200_NVFP4_SUCCESS : B200_NVFP4_CUDA_ERROR;
}

}  // namespace
}  // namespace b200

extern "C" {

size_t b200_nvfp4_ep_record_bytes(int hidden_size, int num_topk) {
  if (hidden_size <= 0 || num_topk <= 0) return 0;
  return static_cast<size_t>(b200::record_bytes(hidden_size, num_topk));
}

int b200_nvfp4_ep_dest_ranks(const void* topk_ids, void* dest, int num_tokens, int num_topk,
                             int experts_per_rank, int world, b200_stream_t stream) {
  if (topk_ids == nullptr || dest == nullptr || num_tokens <= 0 || num_topk <= 0 ||
      experts_per_rank <= 0 || world <= 0 || world > b200::kMaxWorld) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  b200::ep_dest_kernel<<<(num_tokens + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int*>(topk_ids), static_cast<int*>(dest), num_tokens, num_topk,
      experts_per_rank, world);
  b200::count_launch();
  return b200::check_launch();
}

int b200_nvfp4_ep_pack_rows(void* records, const void* x, const void* topk_ids,
                            const void* topk_weights, const void* send_pos, int num_tokens,
                            int hidden_size, int num_topk, int world, int input_is_bf16,
                            b200_stream_t stream) {
  if (records == nullptr || x == nullptr || topk_ids == nullptr || topk_weights == nullptr ||
      send_pos == nullptr || num_tokens <= 0 || hidden_size <= 0 || (hidden_size % 64) != 0 ||
      num_topk <= 0 || world <= 0 || world > b200::kMaxWorld || !b200::aligned16(records) ||
      !b200::aligned16(x)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  const b200::DeviceInfo& dev = b200::current_device_info();
  if (!dev.ok) return B200_NVFP4_CUDA_ERROR;
  const long long groups_per_row = ((hidden_size >> 4) + 31) >> 5;
  long long blocks = (static_cast<long long>(num_tokens) * groups_per_row + 7) / 8;
  const long long max_blocks = static_cast<long long>(dev.sm_count) * 8;
  if (blocks > max_blocks) blocks = max_blocks;
  auto* rec = static_cast<uint8_t*>(records);
  auto* ids = static_cast<const int*>(topk_ids);
  auto* wts = static_cast<const float*>(topk_weights);
  auto* pos = static_cast<const int*>(send_pos);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (input_is_bf16) {
    b200::ep_pack_kernel<true><<<static_cast<int>(blocks), 256, 0, s>>>(rec, x, ids, wts, pos, num_tokens,
                                                                       hidden_size, num_topk, world);
  } else {
    b200::ep_pack_kernel<false><<<static_cast<int>(blocks), 256, 0, s>>>(rec, x, ids, wts, pos, num_tokens,
                                                                        hidden_size, num_topk, world);
  }
  b200::count_launch();
  return b200::check_launch();
}

int b200_nvfp4_ep_unpack_rows(void* x_packed, void* x_scale, void* topk_ids, void* topk_weights,
                              const void* records, int rows, int hidden_size, int num_topk,
                              b200_stream_t stream) {
  if (x_packed == nullptr || x_scale == nullptr || topk_ids == nullptr || topk_weights == nullptr ||
      records == nullptr || rows <= 0 || hidden_size <= 0 || (hidden_size % 64) != 0 ||
      num_topk <= 0 || !b200::aligned16(x_packed) || !b200::aligned16(x_scale) ||
      !b200::aligned16(records)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  const b200::DeviceInfo& dev = b200::current_device_info();
  if (!dev.ok) return B200_NVFP4_CUDA_ERROR;
  int blocks = (rows + 7) / 8;
  const int max_blocks = dev.sm_count * 8;
  if (blocks > max_blocks) blocks = max_blocks;
  b200::ep_unpack_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(x_packed), static_cast<uint8_t*>(x_scale), static_cast<int*>(topk_ids),
      static_cast<float*>(topk_weights), static_cast<const uint8_t*>(records), rows, hidden_size,
      num_topk);
  b200::count_launch();
  return b200::check_launch();
}

}  // extern "C"
