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

// ---------------------------------------------------------------- peer-to-peer hand-off
//
// The same hand-off without a collective library in the data path: every rank owns a receive
// buffer of `world` slots of `slot_rows` records (slot s belongs to source rank s) and a return
// buffer of `world` slots of `slot_rows` FP16 rows (slot r holds what expert rank r sends back),
// both mapped into every peer's address space. The pack kernel stores each record straight into
// the destination rank's slot over NVLink, the return kernel stores each partial row straight
// into its source's slot; counts travel the same way. Nothing is read back to the host and no
// split sizes are needed: the positions inside a slot are the routing positions. The caller
// separates the phases with a cross-GPU barrier (after the dispatch stores, after the return
// stores). All peer accesses are plain global stores; nothing here waits on another GPU.
struct PeerPointers {
  uint8_t* p[kMaxWorld];
};

template <bool kBf16>
__global__ void __launch_bounds__(256)
ep_dispatch_p2p_kernel(PeerPointers peer_records, PeerPointers peer_counts, int* __restrict__ ret_pos,
                       const void* __restrict__ x, const int* __restrict__ topk_ids,
                       const float* __restrict__ topk_weights, const int* __restrict__ send_pos,
                       const int* __restrict__ send_counts, const int* __restrict__ send_cu, int my_rank,
                       int world, int slot_rows, int num_tokens, int hidden, int num_topk) {
  const int lane = threadIdx.x & 31;
  const int nkb = hidden >> 4;
  const int groups_per_row = (nkb + 31) >> 5;
  const long long rb = record_bytes(hidden, num_topk);
  const int payload_bytes = hidden >> 1;
  const long long items = static_cast<long long>(num_tokens) * groups_per_row;
  const int warps_per_block = blockDim.x >> 5;
  if (blockIdx.x == 0 && threadIdx.x < world)   // how many records each destination will find in my slot
    reinterpret_cast<int*>(peer_counts.p[threadIdx.x])[my_rank] = send_counts[threadIdx.x];
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
      const int pos = send_pos[static_cast<long long>(t) * world + r];
      const int k = pos < 0 ? -1 : pos - send_cu[r];          // index inside my slot at rank r
      if (group == 0 && lane == 0) ret_pos[static_cast<long long>(t) * world + r] = k < 0 ? -1 : r * slot_rows + k;
      if (k < 0 || k >= slot_rows) continue;
      uint8_t* rec = peer_records.p[r] + (static_cast<long long>(my_rank) * slot_rows + k) * rb;
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

// Slot rows -> inputs of the routed layer over all world * slot_rows rows: rows a source did not
// fill get expert id -1 in every position, so the routing ignores them.
// Bounded wait for one ready word (written by another GPU with a system-scope release): true once
// *flag has reached `epoch`; after `limit` clock cycles records code | (rank << 8) and gives up.
__device__ __forceinline__ bool wait_ready(const int* flag, int epoch, long long limit, int* error, int code, int rank) {
  const long long start = clock64();
  while (true) {
    int seen;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
    if (seen - epoch >= 0) return true;
    if (clock64() - start > limit) {
      if (error != nullptr) atomicCAS(error, 0, code | (rank << 8));
      return false;
    }
    __nanosleep(64);
  }
}

constexpr int kDispatchNotReadyCode = 10;
constexpr int kReturnNotReadyCode = 11;

// With `ready` != nullptr a warp takes up the rows of source rank s only once ready[s] has reached
// `epoch` (the source publishes it after its dispatch stores): rows of sources that have already
// delivered are unpacked while others are still on their way. A source that never becomes ready
// leaves its rows marked empty and a code in the device error word.
__global__ void __launch_bounds__(256)
ep_unpack_slots_kernel(uint8_t* __restrict__ x_packed, uint8_t* __restrict__ x_scale, int* __restrict__ ids,
                       float* __restrict__ weights, const uint8_t* records, const int* counts, int world,
                       int slot_rows, int hidden, int num_topk, const int* ready, int epoch, long long limit,
                       int* error) {
  // records and counts are written by other GPUs while this kernel waits: plain (coherent) loads
  // after the acquire of the ready word, no read-only-cache path.
  const int lane = threadIdx.x & 31;
  const int nkb = hidden >> 4;
  const int kt = (nkb + 3) >> 2;
  const long long rb = record_bytes(hidden, num_topk);
  const int payload_bytes = hidden >> 1;
  const int warps_per_block = blockDim.x >> 5;
  const int rows = world * slot_rows;
  unsigned long long seen_ready = 0, seen_late = 0;      // per warp, one bit per source rank (world <= 64)
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const int src_rank = row / slot_rows;
    bool arrived = true;
    if (ready != nullptr) {
      // one acquire per warp and source: a source this warp has seen ready stays ready, and one that
      // ran into the limit is not waited for again (a dead source costs a warp one time-out, not one
      // per row)
      const unsigned long long bit = 1ull << src_rank;
      if ((seen_ready & bit) == 0 && (seen_late & bit) == 0) {
        int ok = 1;
        if (lane == 0) ok = wait_ready(ready + src_rank, epoch, limit, error, kDispatchNotReadyCode, src_rank) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok != 0) seen_ready |= bit; else seen_late |= bit;
      }
      arrived = (seen_ready & bit) != 0;
    }
    const bool valid = arrived && row - src_rank * slot_rows < counts[src_rank];
    if (!valid) {
      for (int j = lane; j < num_topk; j += 32) {
        ids[static_cast<long long>(row) * num_topk + j] = -1;
        weights[static_cast<long long>(row) * num_topk + j] = 0.0f;
      }
      continue;
    }
    const uint8_t* rec = records + static_cast<long long>(row) * rb;
    const uint4* src = reinterpret_cast<const uint4*>(rec);
    uint4* dst = reinterpret_cast<uint4*>(x_packed + static_cast<long long>(row) * payload_bytes);
    for (int i = lane; i < (payload_bytes >> 4); i += 32) dst[i] = src[i];
    uint8_t* s_row = x_scale + sf_offset(row, 0, kt);
    for (int j = lane; j < kt; j += 32)
      *reinterpret_cast<uint32_t*>(s_row + static_cast<long long>(j) * 512) =
          *reinterpret_cast<const uint32_t*>(rec + payload_bytes + 4 * j);
    const int* rid = reinterpret_cast<const int*>(rec + payload_bytes + nkb);
    const float* rw = reinterpret_cast<const float*>(rec + payload_bytes + nkb + 4 * num_topk);
    for (int j = lane; j < num_topk; j += 32) {
      ids[static_cast<long long>(row) * num_topk + j] = rid[j];
      weights[static_cast<long long>(row) * num_topk + j] = rw[j];
    }
  }
}

// Partial rows back to their sources: row (s, k) of my slots goes to row (my_rank, k) of rank s.
__global__ void __launch_bounds__(256)
ep_return_p2p_kernel(PeerPointers peer_ret, const uint8_t* __restrict__ partial, const int* __restrict__ counts,
                     int my_rank, int world, int slot_rows, int row_bytes) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int rows = world * slot_rows;
  const int vecs = row_bytes >> 4;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const int src_rank = row / slot_rows;
    const int k = row - src_rank * slot_rows;
    if (k >= counts[src_rank]) continue;
    const uint4* s4 = reinterpret_cast<const uint4*>(partial + static_cast<long long>(row) * row_bytes);
    uint4* d4 = reinterpret_cast<uint4*>(peer_ret.p[src_rank] +
                                         (static_cast<long long>(my_rank) * slot_rows + k) * row_bytes);
    for (int v = lane; v < vecs; v += 32) d4[v] = s4[v];
  }
}

// The weighted sum over a received token's local experts (the reduce step of the routed layer,
// src/fused_moe/reduce.cu:12-35: FP32 accumulation in route order, one rounding to FP16) for one
// 16-byte chunk of a slot row: eight FP16 values packed. (Issuing the loads of all local routes
// before the first FMA was measured and is slower here: most routes of a received row belong to
// other ranks.)
__device__ __forceinline__ uint4 reduce_chunk(const __half* __restrict__ down_output, const int* __restrict__ pos,
                                              const float* __restrict__ wts, int num_topk, int hidden, int col) {
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  for (int r = 0; r < num_topk; ++r) {
    const int drow = pos[r];
    if (drow < 0) continue;
    const float wt = wts[r];
    const uint4 d = *reinterpret_cast<const uint4*>(down_output + static_cast<long long>(drow) * hidden + col);
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
    const __half2 h = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
    ow[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return o;
}

// Partial rows written straight into the source ranks' return slots instead of a local matrix:
// row (s, k) of the slot space -> row (my_rank, k) of rank s, over the column window
// [col_start, col_start + col_count). Rows beyond a slot's count are skipped. One thread per
// 16-byte chunk, one plain 16-byte store into the peer's memory (handing 4 KB pieces to the bulk-copy
// engine from shared memory instead was measured and is slower: 0.28 against 0.18 ms on 4 GPUs).
__global__ void __launch_bounds__(256)
ep_reduce_return_p2p_kernel(PeerPointers peer_ret, const __half* __restrict__ down_output,
                            const int* __restrict__ topk_pos, const float* __restrict__ topk_scale,
                            const int* __restrict__ counts, int my_rank, int world, int slot_rows, int hidden,
                            int num_topk, int col_start, int col_count) {
  const int chunks = col_count >> 3;
  const long long items = static_cast<long long>(world) * slot_rows * chunks;
  for (long long item = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; item < items;
       item += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(item / chunks);
    const int col = col_start + static_cast<int>(item % chunks) * 8;
    const int src_rank = row / slot_rows;
    const int k = row - src_rank * slot_rows;
    if (k >= counts[src_rank]) continue;
    const uint4 o = reduce_chunk(down_output, topk_pos + static_cast<long long>(row) * num_topk,
                                 topk_scale + static_cast<long long>(row) * num_topk, num_topk, hidden, col);
    __half* dst = reinterpret_cast<__half*>(peer_ret.p[src_rank]) +
                  (static_cast<long long>(my_rank) * slot_rows + k) * hidden + col;
    *reinterpret_cast<uint4*>(dst) = o;
  }
}

// Cross-GPU barrier of the peer-memory transport. Every rank owns `world` flag words in its
// symmetric buffer; flag s of rank r is written by rank s only. Thread r of the one block stores
// this call's epoch into flag `my_rank` of rank r (after a system-scope fence, so the peer stores
// of the kernels before it on the stream are visible first), then waits until its own flag r has
// reached the epoch. The wait is bounded: after `limit_cycles` it records
// kBarrierTimeoutCode | (late rank << 8) in the device error word and returns, so a rank that
// is late, failed or gone costs the others one time-out instead of an endless spin. Epochs only
// grow (signed difference compare, so the counter may wrap).
constexpr int kBarrierTimeoutCode = 9;

__global__ void __launch_bounds__(kMaxWorld)
ep_barrier_kernel(PeerPointers peer_flags, int my_rank, int world, int epoch, long long limit_cycles,
                  int* __restrict__ error) {
  const int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();
    int* remote = reinterpret_cast<int*>(peer_flags.p[r]) + my_rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const int* local = reinterpret_cast<const int*>(peer_flags.p[my_rank]) + r;
    const long long start = clock64();
    while (true) {
      int seen;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(local) : "memory");
      if (seen - epoch >= 0) break;
      if (clock64() - start > limit_cycles) {
        if (error != nullptr) atomicCAS(error, 0, kBarrierTimeoutCode | (r << 8));
        break;
      }
      __nanosleep(64);
    }
    __threadfence_system();
  }
}

// The publishing half of the barrier alone: tells every peer that this rank's stores of the
// kernels before it on the stream are complete (system-scope fence, then the epoch into word
// `slot + my_rank` of every peer's flag array). Nothing waits here; the consumers do, per source.
__global__ void __launch_bounds__(kMaxWorld)
ep_publish_kernel(PeerPointers peer_flags, int my_rank, int world, int slot, int epoch) {
  const int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();
    int* remote = reinterpret_cast<int*>(peer_flags.p[r]) + slot + my_rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  }
}

// Final step at the source: out[t] = sum over ranks r (ascending) of the partial row rank r stored
// into this rank's return slots, FP32 accumulation, one rounding - b200_nvfp4_moe_reduce with unit
// weights - after a bounded wait until every rank has published its return stores of this epoch.
template <bool kOutBf16>
__global__ void __launch_bounds__(256)
ep_sum_kernel(void* __restrict__ output, const __half* ret, const int* __restrict__ ret_pos,
              int num_tokens, int hidden, int world, const int* ready, int epoch, long long limit, int* error) {
  if (ready != nullptr) {
    if (threadIdx.x < world) wait_ready(ready + threadIdx.x, epoch, limit, error, kReturnNotReadyCode, threadIdx.x);
    __syncthreads();
  }
  const int chunks = hidden >> 3;
  const long long items = static_cast<long long>(num_tokens) * chunks;
  for (long long item = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; item < items;
       item += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int token = static_cast<int>(item / chunks);
    const int col = static_cast<int>(item % chunks) * 8;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
    const int* pos = ret_pos + static_cast<long long>(token) * world;
    for (int r = 0; r < world; ++r) {
      const int row = pos[r];
      if (row < 0) continue;
      const uint4 d = *reinterpret_cast<const uint4*>(ret + static_cast<long long>(row) * hidden + col);
      const uint32_t w[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
        acc[2 * i] = __fmaf_rn(__low2float(h), 1.0f, acc[2 * i]);
        acc[2 * i + 1] = __fmaf_rn(__high2float(h), 1.0f, acc[2 * i + 1]);
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

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

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
  return b200::launch_status();
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
  return b200::launch_status();
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
  return b200::launch_status();
}

int b200_nvfp4_ep_dispatch_p2p(const void* const* peer_records, const void* const* peer_counts, void* ret_pos,
                               const void* x, const void* topk_ids, const void* topk_weights,
                               const void* send_pos, const void* send_counts, const void* send_cu, int my_rank,
                               int world, int slot_rows, int num_tokens, int hidden_size, int num_topk,
                               int input_is_bf16, b200_stream_t stream) {
  if (peer_records == nullptr || peer_counts == nullptr || ret_pos == nullptr || x == nullptr ||
      topk_ids == nullptr || topk_weights == nullptr || send_pos == nullptr || send_counts == nullptr ||
      send_cu == nullptr || world <= 0 || world > b200::kMaxWorld || my_rank < 0 || my_rank >= world ||
      slot_rows <= 0 || num_tokens <= 0 || num_tokens > slot_rows || hidden_size <= 0 ||
      (hidden_size % 64) != 0 || num_topk <= 0 || !b200::aligned16(x)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  b200::PeerPointers rec{}, cnt{};
  for (int r = 0; r < world; ++r) {
    if (peer_records[r] == nullptr || peer_counts[r] == nullptr || !b200::aligned16(peer_records[r]))
      return B200_NVFP4_INVALID_ARGUMENT;
    rec.p[r] = static_cast<uint8_t*>(const_cast<void*>(peer_records[r]));
    cnt.p[r] = static_cast<uint8_t*>(const_cast<void*>(peer_counts[r]));
  }
  const b200::DeviceInfo& dev = b200::current_device_info();
  if (!dev.ok) return B200_NVFP4_CUDA_ERROR;
  const long long groups_per_row = ((hidden_size >> 4) + 31) >> 5;
  long long blocks = (static_cast<long long>(num_tokens) * groups_per_row + 7) / 8;
  const long long max_blocks = static_cast<long long>(dev.sm_count) * 8;
  if (blocks > max_blocks) blocks = max_blocks;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto* ids = static_cast<const int*>(topk_ids);
  auto* wts = static_cast<const float*>(topk_weights);
  if (input_is_bf16) {
    b200::ep_dispatch_p2p_kernel<true><<<static_cast<int>(blocks), 256, 0, s>>>(
        rec, cnt, static_cast<int*>(ret_pos), x, ids, wts, static_cast<const int*>(send_pos),
        static_cast<const int*>(send_counts), static_cast<const int*>(send_cu), my_rank, world, slot_rows,
        num_tokens, hidden_size, num_topk);
  } else {
    b200::ep_dispatch_p2p_kernel<false><<<static_cast<int>(blocks), 256, 0, s>>>(
        rec, cnt, static_cast<int*>(ret_pos), x, ids, wts, static_cast<const int*>(send_pos),
        static_cast<const int*>(send_counts), static_cast<const int*>(send_cu), my_rank, world, slot_rows,
        num_tokens, hidden_size, num_topk);
  }
  b200::count_launch();
  return b200::launch_status();
}

int b200_nvfp4_ep_unpack_slots(void* x_packed, void* x_scale, void* topk_ids, void* topk_weights,
                               const void* records, const void* counts, int world, int slot_rows,
                               int hidden_size, int num_topk, b200_stream_t stream) {
  return b200_nvfp4_ep_unpack_slots_ready(x_packed, x_scale, topk_ids, topk_weights, records, counts, world,
                                          slot_rows, hidden_size, num_topk, nullptr, 0, 0, stream);
}

int b200_nvfp4_ep_unpack_slots_ready(void* x_packed, void* x_scale, void* topk_ids, void* topk_weights,
                                     const void* records, const void* counts, int world, int slot_rows,
                                     int hidden_size, int num_topk, const void* ready, int epoch,
                                     long long limit_cycles, b200_stream_t stream) {
  if (limit_cycles < 0 || (ready != nullptr && (reinterpret_cast<uintptr_t>(ready) & 3u) != 0))
    return B200_NVFP4_INVALID_ARGUMENT;
  if (x_packed == nullptr || x_scale == nullptr || topk_ids == nullptr || topk_weights == nullptr ||
      records == nullptr || counts == nullptr || world <= 0 || world > b200::kMaxWorld || slot_rows <= 0 ||
      hidden_size <= 0 || (hidden_size % 64) != 0 || num_topk <= 0 || !b200::aligned16(x_packed) ||
      !b200::aligned16(x_scale) || !b200::aligned16(records)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  const b200::DeviceInfo& dev = b200::current_device_info();
  if (!dev.ok) return B200_NVFP4_CUDA_ERROR;
  long long blocks = (static_cast<long long>(world) * slot_rows + 7) / 8;
  const long long max_blocks = static_cast<long long>(dev.sm_count) * 8;
  if (blocks > max_blocks) blocks = max_blocks;
  b200::ep_unpack_slots_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(x_packed), static_cast<uint8_t*>(x_scale), static_cast<int*>(topk_ids),
      static_cast<float*>(topk_weights), static_cast<const uint8_t*>(records), static_cast<const int*>(counts),
      world, slot_rows, hidden_size, num_topk, static_cast<const int*>(ready), epoch,
      limit_cycles > 0 ? limit_cycles : (1ll << 31), b200::device_error_word());
  b200::count_launch();
  return b200::launch_status();
}

int b200_nvfp4_ep_return_p2p(const void* const* peer_ret, const void* partial, const void* counts, int my_rank,
                             int world, int slot_rows, int row_bytes, b200_stream_t stream) {
  if (peer_ret == nullptr || partial == nullptr || counts == nullptr || world <= 0 ||
      world > b200::kMaxWorld || my_rank < 0 || my_rank >= world || slot_rows <= 0 || row_bytes <= 0 ||
      (row_bytes % 16) != 0 || !b200::aligned16(partial)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  b200::PeerPointers ret{};
  for (int r = 0; r < world; ++r) {
    if (peer_ret[r] == nullptr || !b200::aligned16(peer_ret[r])) return B200_NVFP4_INVALID_ARGUMENT;
    ret.p[r] = static_cast<uint8_t*>(const_cast<void*>(peer_ret[r]));
  }
  const b200::DeviceInfo& dev = b200::current_device_info();
  if (!dev.ok) return B200_NVFP4_CUDA_ERROR;
  long long blocks = (static_cast<long long>(world) * slot_rows + 7) / 8;
  const long long max_blocks = static_cast<long long>(dev.sm_count) * 8;
  if (blocks > max_blocks) blocks = max_blocks;
  b200::ep_return_p2p_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      ret, static_cast<const uint8_t*>(partial), static_cast<const int*>(counts), my_rank, world, slot_rows,
      row_bytes);
  b200::count_launch();
  return b200::launch_status();
}

int b200_nvfp4_ep_reduce_return_p2p(const void* const* peer_ret, const void* down_output, const void* topk_pos,
                                    const void* topk_scale, const void* counts, int my_rank, int world,
                                    int slot_rows, int hidden_size, int num_topk, b200_stream_t stream) {
  return b200_nvfp4_ep_reduce_return_p2p_columns(peer_ret, down_output, topk_pos, topk_scale, counts, my_rank,
                                                 world, slot_rows, hidden_size, num_topk, 0, hidden_size, stream);
}

int b200_nvfp4_ep_reduce_return_p2p_columns(const void* const* peer_ret, const void* down_output,
                                            const void* topk_pos, const void* topk_scale, const void* counts,
                                            int my_rank, int world, int slot_rows, int hidden_size, int num_topk,
                                            int col_start, int col_count, b200_stream_t stream) {
  if (col_start < 0 || col_count <= 0 || (col_start % 8) != 0 || (col_count % 8) != 0 ||
      col_start > hidden_size - col_count) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  if (peer_ret == nullptr || down_output == nullptr || topk_pos == nullptr || topk_scale == nullptr ||
      counts == nullptr || world <= 0 || world > b200::kMaxWorld || my_rank < 0 || my_rank >= world ||
      slot_rows <= 0 || hidden_size <= 0 || (hidden_size % 8) != 0 || num_topk <= 0 ||
      !b200::aligned16(down_output)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  b200::PeerPointers ret{};
  for (int r = 0; r < world; ++r) {
    if (peer_ret[r] == nullptr || !b200::aligned16(peer_ret[r])) return B200_NVFP4_INVALID_ARGUMENT;
    ret.p[r] = static_cast<uint8_t*>(const_cast<void*>(peer_ret[r]));
  }
  const b200::DeviceInfo& dev = b200::current_device_info();
  if (!dev.ok) return B200_NVFP4_CUDA_ERROR;
  const long long items = static_cast<long long>(world) * slot_rows * (col_count >> 3);
  long long blocks = (items + 255) / 256;
  const long long max_blocks = static_cast<long long>(dev.sm_count) * 16;
  if (blocks > max_blocks) blocks = max_blocks;
  b200::ep_reduce_return_p2p_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      ret, static_cast<const __half*>(down_output), static_cast<const int*>(topk_pos),
      static_cast<const float*>(topk_scale), static_cast<const int*>(counts), my_rank, world, slot_rows,
      hidden_size, num_topk, col_start, col_count);
  b200::count_launch();
  return b200::launch_status();
}

int b200_nvfp4_ep_barrier_p2p(const void* const* peer_flags, int my_rank, int world, int epoch,
                              long long limit_cycles, b200_stream_t stream) {
  if (peer_flags == nullptr || world <= 0 || world > b200::kMaxWorld || my_rank < 0 || my_rank >= world ||
      limit_cycles < 0) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  b200::PeerPointers flags{};
  for (int r = 0; r < world; ++r) {
    if (peer_flags[r] == nullptr || (reinterpret_cast<uintptr_t>(peer_flags[r]) & 3u) != 0)
      return B200_NVFP4_INVALID_ARGUMENT;
    flags.p[r] = static_cast<uint8_t*>(const_cast<void*>(peer_flags[r]));
  }
  int* error = b200::device_error_word();
  if (error == nullptr) return B200_NVFP4_CUDA_ERROR;
  const long long limit = limit_cycles > 0 ? limit_cycles : (1ll << 31);   // about a second
  b200::ep_barrier_kernel<<<1, b200::kMaxWorld, 0, static_cast<cudaStream_t>(stream)>>>(flags, my_rank, world, epoch,
                                                                                     limit, error);
  b200::count_launch();
  return b200::launch_status();
}

int b200_nvfp4_ep_publish_p2p(const void* const* peer_flags, int my_rank, int world, int slot, int epoch,
                              b200_stream_t stream) {
  if (peer_flags == nullptr || world <= 0 || world > b200::kMaxWorld || my_rank < 0 || my_rank >= world || slot < 0)
    return B200_NVFP4_INVALID_ARGUMENT;
  b200::PeerPointers flags{};
  for (int r = 0; r < world; ++r) {
    if (peer_flags[r] == nullptr || (reinterpret_cast<uintptr_t>(peer_flags[r]) & 3u) != 0)
      return B200_NVFP4_INVALID_ARGUMENT;
    flags.p[r] = static_cast<uint8_t*>(const_cast<void*>(peer_flags[r]));
  }
  b200::ep_publish_kernel<<<1, b200::kMaxWorld, 0, static_cast<cudaStream_t>(stream)>>>(flags, my_rank, world, slot, epoch);
  b200::count_launch();
  return b200::launch_status();
}

int b200_nvfp4_ep_sum_p2p(void* output, const void* ret, const void* ret_pos, int num_tokens, int hidden_size,
                          int world, int out_is_bf16, const void* ready, int epoch, long long limit_cycles,
                          b200_stream_t stream) {
  if (output == nullptr || ret == nullptr || ret_pos == nullptr || num_tokens <= 0 || hidden_size <= 0 ||
      (hidden_size % 8) != 0 || world <= 0 || world > b200::kMaxWorld || limit_cycles < 0 ||
      !b200::aligned16(output) || !b200::aligned16(ret) || (ready != nullptr && (reinterpret_cast<uintptr_t>(ready) & 3u) != 0)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  const b200::DeviceInfo& dev = b200::current_device_info();
  if (!dev.ok) return B200_NVFP4_CUDA_ERROR;
  const long long items = static_cast<long long>(num_tokens) * (hidden_size >> 3);
  long long blocks = (items + 255) / 256;
  const long long max_blocks = static_cast<long long>(dev.sm_count) * 16;
  if (blocks > max_blocks) blocks = max_blocks;
  const long long limit = limit_cycles > 0 ? limit_cycles : (1ll << 31);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_is_bf16)
    b200::ep_sum_kernel<true><<<static_cast<int>(blocks), 256, 0, s>>>(
        output, static_cast<const __half*>(ret), static_cast<const int*>(ret_pos), num_tokens, hidden_size, world,
        static_cast<const int*>(ready), epoch, limit, b200::device_error_word());
  else
    b200::ep_sum_kernel<false><<<static_cast<int>(blocks), 256, 0, s>>>(
        output, static_cast<const __half*>(ret), static_cast<const int*>(ret_pos), num_tokens, hidden_size, world,
        static_cast<const int*>(ready), epoch, limit, b200::device_error_word());
  b200::count_launch();
  return b200::launch_status();
}

}  // extern "C"
