// Persistent, warp-specialised NVFP4 block-scaled GEMM for sm_100a.
//
//   Y[g][r, c] = alpha_g * sum_k (A[g][r,k] * SFA[g][r,k/16]) * (B[g][c,k] * SFB[g][c,k/16])
//
// A and B are packed E2M1 (two values per byte, K contiguous), SFA/SFB are UE4M3 bytes in
// the 512-byte-atom block-scaled layout (128 rows x 4 k-blocks per atom, atoms K-major
// inside a 128-row tile). One kernel serves the single GEMM, the strided-batched GEMM, the
// split-K partial pass and the expert-grouped GEMM: a "group" is a set of rows of A with
// its own B matrix and scale regions, and the row ranges come either from constants
// (dense / batched) or from device arrays seqlens / cu_seqlens (grouped).
//
// Replaces, from the reference: nvfp4_gemm_kernel (src/gemm/cute_gemm.cu:21-321),
// nvfp4_m128_partial_kernel / nvfp4_m256_partial_kernel
// (src/gemm/specialized/m128_gemm.cu:43-365), group_gemm_nvfp4_kernel and its four
// set-up kernels (src/grouped_gemm/kernels.cuh:66-449).
//
// Structure of one CTA (192 threads, one CTA per SM):
//   warp 0      producer: TMA loads of the A / B tiles (128-byte swizzle) and untiled bulk
//               copies of the scale atoms into a ring of shared-memory stages
//   warp 1      MMA issuer: tcgen05.cp moves scale atoms shared -> tensor memory, then
//               tcgen05.mma kind::mxf4nvf4 (128 x BN x 64 per instruction) accumulates FP32
//               in tensor memory; tcgen05.commit releases the stage / publishes the tile
//   warps 2-5   epilogue: tcgen05.ld of the accumulator (one 32-lane quarter per warp),
//               conversion, staging through shared memory, coalesced 16-byte stores with
//               row / column predicates
// All mbarrier waits are bounded (ptx::mbar_wait); a timeout is reported through
// GemmParams::error instead of hanging.
#pragma once

#include <cuda_fp16.h>

#include "ptx.cuh"

namespace b200 {

constexpr int kBlockM = 128;        // rows of A per tile = UMMA M
constexpr int kStageKBytes = 128;   // bytes of K per stage row = one swizzle span
constexpr int kStageK = 256;        // E2M1 values of K per stage
constexpr int kAtomBytes = 512;     // one scale atom: 128 rows x 4 k-blocks
constexpr int kMaxGroups = 1024;
constexpr int kGemmThreads = 192;
constexpr int kStagingRowBytes = 144;  // 128 payload bytes + 16 pad: conflict-free 16-byte rows
constexpr int kStagingBytes = 4 * 32 * kStagingRowBytes;
constexpr int kSmemBudget = 232448;  // 227 KB opt-in limit per CTA

struct GemmParams {
  int num_groups;
  int n;                      // output columns per group
  int k;                      // logical K
  int m_uniform;              // rows per group when seqlens == nullptr
  const int* seqlens;         // [G] valid rows per group (device) or nullptr
  const int* cu_seqlens;      // [G+1] first row of each group (device) or nullptr
  const uint8_t* sfa;
  const uint8_t* sfb;
  long long sfa_group_stride;  // bytes between the scale regions of consecutive groups
  long long sfb_group_stride;
  int b_group_rows;           // rows of B per group (N), 0 when every group shares one B
  void* out;                  // FP16 or FP32 [rows, n]
  long long out_split_stride;  // elements between split-K slices of `out`
  const float* group_alpha;   // optional per-group multiplier applied in FP32
  int num_splits;             // split-K factor (1 = none)
  int raster_m;               // m-tiles per rasterisation band
  int* tiles_out;             // optional [G]   ceil(rows/128) per group
  int* cu_tiles_out;          // optional [G+1] exclusive prefix of tiles_out
  int* error;                 // device word that receives a non-zero code on a timed-out wait
};

template <int BN>
struct GemmCfg {
  static_assert(BN == 32 || BN == 64 || BN == 128 || BN == 256, "unsupported tile width");
  static constexpr int kSfbGroups = (BN + 127) / 128;       // 128-row scale tiles per B tile
  static constexpr int kSfbColsPerMma = 4 * kSfbGroups;     // TMEM columns of SFB per MMA
  static constexpr int kAccStages = BN <= 128 ? 2 : 1;
  static constexpr int kSfaCol = kAccStages * BN;
  static constexpr int kSfbCol = kSfaCol + 16;
  static constexpr int kUsedCols = kSfbCol + 4 * kSfbColsPerMma;
  static constexpr int kTmemCols = kUsedCols <= 128 ? 128 : (kUsedCols <= 256 ? 256 : 512);
  static constexpr int kABytes = kBlockM * kStageKBytes;
  static constexpr int kBBytes = BN * kStageKBytes;
  static constexpr int kSfaBytes = 4 * kAtomBytes;
  static constexpr int kSfbBytes = kSfbGroups * 4 * kAtomBytes;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kFixedBytes = 1024 /*alignment slack*/ + kStagingBytes + 256 /*barriers*/ +
                                     3 * (kMaxGroups + 1) * 4;
  static constexpr int kStagesRaw = (kSmemBudget - kFixedBytes) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kSmemBytes = kFixedBytes + kStages * kStageBytes;
  static_assert(kStages >= 3, "pipeline too shallow");
};

struct TileCoord {
  int g, mt, nt, split;
};

// Flat task id -> (group, m-tile inside the group, n-tile, k-split). m-tiles of all groups
// are numbered consecutively; bands of `raster_m` m-tiles sweep the n-tiles so CTAs that
// run at the same time share A rows and B columns in L2.
__device__ __forceinline__ TileCoord decode_tile(int task, int total_mt, int n_tiles,
                                                 int num_splits, int raster_m,
                                                 const int* s_cu_tiles, int num_groups) {
  TileCoord t;
  t.split = task % num_splits;
  int flat = task / num_splits;
  int per_band = raster_m * n_tiles;
  int band = flat / per_band;
  int first = band * raster_m;
  int band_m = min(raster_m, total_mt - first);
  int rem = flat - band * per_band;
  int mtt = first + rem % band_m;
  t.nt = rem / band_m;
  int lo = 0, hi = num_groups;  // largest g with s_cu_tiles[g] <= mtt (skips empty groups)
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (s_cu_tiles[mid] <= mtt) lo = mid; else hi = mid;
  }
  t.g = lo;
  t.mt = mtt - s_cu_tiles[lo];
  return t;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int BN, bool kOutF32>
__global__ void __launch_bounds__(kGemmThreads, 1)
nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                  const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kAccStages = Cfg::kAccStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* stage_base = smem;
  uint8_t* staging = smem + kStages * Cfg::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + kStagingBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* acc_full_bar = empty_bar + kStages;
  uint64_t* acc_empty_bar = acc_full_bar + kAccStages;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty_bar + kAccStages);
  int* abort_flag = reinterpret_cast<int*>(tmem_holder + 1);
  int* s_cu_tiles = reinterpret_cast<int*>(staging + kStagingBytes + 256);
  int* s_row0 = s_cu_tiles + (p.num_groups + 1);
  int* s_rows = s_row0 + (p.num_groups + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int G = p.num_groups;

  // ---- group tables: valid rows, first row and m-tile prefix of every group
  for (int g = threadIdx.x; g < G; g += kGemmThreads) {
    int rows = p.seqlens ? p.seqlens[g] : p.m_uniform;
    rows = rows > 0 ? rows : 0;
    s_rows[g] = rows;
    s_row0[g] = p.cu_seqlens ? p.cu_seqlens[g] : g * p.m_uniform;
    s_cu_tiles[g] = (rows + kBlockM - 1) / kBlockM;
  }
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar + s, 1);
      ptx::mbar_init(empty_bar + s, 1);
    }
    for (int s = 0; s < kAccStages; ++s) {
      ptx::mbar_init(acc_full_bar + s, 1);
      ptx::mbar_init(acc_empty_bar + s, 4);
    }
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
  }
  __syncthreads();
  if (warp == 0) {  // exclusive scan of the per-group tile counts, 32 groups at a time
    int carry = 0;
    for (int base = 0; base < G; base += 32) {
      int v = (base + lane < G) ? s_cu_tiles[base + lane] : 0;
      int incl = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        int o = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += o;
      }
      if (base + lane < G) {
        if (blockIdx.x == 0 && p.tiles_out) p.tiles_out[base + lane] = v;
        if (blockIdx.x == 0 && p.cu_tiles_out) p.cu_tiles_out[base + lane] = carry + incl - v;
        s_cu_tiles[base + lane] = carry + incl - v;
      }
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      s_cu_tiles[G] = carry;
      if (blockIdx.x == 0 && p.cu_tiles_out) p.cu_tiles_out[G] = carry;
    }
  } else if (warp == 1) {
    ptx::tmem_alloc(tmem_holder, Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();

  const uint32_t tmem_base = *tmem_holder;
  const int total_mt = s_cu_tiles[G];
  const int n_tiles = (p.n + BN - 1) / BN;
  const int total_tasks = total_mt * n_tiles * p.num_splits;
  const int kt = (p.k + 63) / 64;               // scale atoms along K
  const int k_stages = (kt + 3) / 4;            // pipeline stages along K
  const int n_sf_tiles = (p.n + 127) / 128;     // 128-row scale tiles of B

  if (warp == 0) {
    // =============================== producer ===============================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int task = blockIdx.x; task < total_tasks && ok; task += gridDim.x) {
        TileCoord t = decode_tile(task, total_mt, n_tiles, p.num_splits, p.raster_m, s_cu_tiles, G);
        const int a_row = s_row0[t.g] + t.mt * kBlockM;
        const int b_row = t.g * p.b_group_rows + t.nt * BN;
        const uint8_t* sfa_tile = p.sfa + t.g * p.sfa_group_stride +
                                  static_cast<long long>(t.mt) * kt * kAtomBytes;
        const int sf_tile0 = (t.nt * BN) / 128;
        const uint8_t* sfb_tile = p.sfb + t.g * p.sfb_group_stride +
                                  static_cast<long long>(sf_tile0) * kt * kAtomBytes;
        int sfb_groups = Cfg::kSfbGroups;
        if (sf_tile0 + sfb_groups > n_sf_tiles) sfb_groups = n_sf_tiles - sf_tile0;
        const int ks_begin = (k_stages * t.split) / p.num_splits;
        const int ks_end = (k_stages * (t.split + 1)) / p.num_splits;
        for (int ks = ks_begin; ks < ks_end; ++ks) {
          if (!ptx::mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, 1)) { ok = false; break; }
          uint8_t* sa = stage_base + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          uint8_t* ssfa = sb + Cfg::kBBytes;
          uint8_t* ssfb = ssfa + Cfg::kSfaBytes;
          const int atoms = min(4, kt - ks * 4);
          const uint32_t sf_bytes = static_cast<uint32_t>(atoms) * kAtomBytes;
          ptx::mbar_arrive_expect_tx(full_bar + stage,
                                     Cfg::kABytes + Cfg::kBBytes + sf_bytes * (1 + sfb_groups));
          ptx::tma_load_2d(sa, &tmap_a, full_bar + stage, ks * kStageKBytes, a_row);
          ptx::tma_load_2d(sb, &tmap_b, full_bar + stage, ks * kStageKBytes, b_row);
          ptx::bulk_load(ssfa, sfa_tile + static_cast<long long>(ks) * 4 * kAtomBytes, sf_bytes,
                         full_bar + stage);
          for (int gi = 0; gi < sfb_groups; ++gi)
            ptx::bulk_load(ssfb + gi * 4 * kAtomBytes,
                           sfb_tile + (static_cast<long long>(gi) * kt + ks * 4) * kAtomBytes,
                           sf_bytes, full_bar + stage);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // =============================== MMA issuer ==============================
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_idesc_nvfp4(kBlockM, BN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int task = blockIdx.x; task < total_tasks && ok; task += gridDim.x) {
        TileCoord t = decode_tile(task, total_mt, n_tiles, p.num_splits, p.raster_m, s_cu_tiles, G);
        const int ks_begin = (k_stages * t.split) / p.num_splits;
        const int ks_end = (k_stages * (t.split + 1)) / p.num_splits;
        // A tile narrower than 128 columns uses part of a 128-row scale atom: column
        // (n0 % 128) / 32 of the four TMEM columns the atom occupies.
        const uint32_t sfb_sub = BN < 128 ? static_cast<uint32_t>(((t.nt * BN) % 128) / 32) : 0u;
        if (!ptx::mbar_wait(acc_empty_bar + acc, acc_phase ^ 1, abort_flag, 2)) break;
        ptx::tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int ks = ks_begin; ks < ks_end; ++ks) {
          if (!ptx::mbar_wait(full_bar + stage, phase, abort_flag, 3)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          uint8_t* sa = stage_base + stage * Cfg::kStageBytes;
          const uint32_t a_addr = ptx::smem_u32(sa);
          const uint32_t b_addr = a_addr + Cfg::kABytes;
          const uint32_t sfa_addr = b_addr + Cfg::kBBytes;
          const uint32_t sfb_addr = sfa_addr + Cfg::kSfaBytes;
          const int atoms = min(4, kt - ks * 4);
          for (int j = 0; j < atoms; ++j) {
            ptx::tc_cp_32x128b_warpx4(tmem_base + Cfg::kSfaCol + 4 * j,
                                      ptx::make_sf_desc(sfa_addr + j * kAtomBytes));
#pragma unroll
            for (int gi = 0; gi < Cfg::kSfbGroups; ++gi)
              ptx::tc_cp_32x128b_warpx4(
                  tmem_base + Cfg::kSfbCol + j * Cfg::kSfbColsPerMma + 4 * gi,
                  ptx::make_sf_desc(sfb_addr + (gi * 4 + j) * kAtomBytes));
          }
          const uint64_t a_desc = ptx::make_kmajor_sw128_desc(a_addr);
          const uint64_t b_desc = ptx::make_kmajor_sw128_desc(b_addr);
          for (int j = 0; j < atoms; ++j) {
            // 64 E2M1 values = 32 bytes along K: +2 in the descriptor's 16-byte address field
            ptx::tc_mma_nvfp4(tmem_acc, a_desc + 2 * j, b_desc + 2 * j, idesc,
                              tmem_base + Cfg::kSfaCol + 4 * j,
                              tmem_base + Cfg::kSfbCol + j * Cfg::kSfbColsPerMma + sfb_sub,
                              (ks > ks_begin || j > 0) ? 1u : 0u);
          }
          ptx::tc_commit(empty_bar + stage);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        ptx::tc_commit(acc_full_bar + acc);
        if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // ================================ epilogue ===============================
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    uint8_t* my_staging = staging + (warp - 2) * 32 * kStagingRowBytes;
    constexpr int kChunkCols = kOutF32 ? 32 : (BN < 64 ? BN : 64);   // columns per store pass
    constexpr int kChunkBytes = kChunkCols * (kOutF32 ? 4 : 2);
    constexpr int kLanesPerRow = kChunkBytes / 16;
    constexpr int kRowsPerPass = 32 / kLanesPerRow;
    constexpr int kElemsPer16B = kOutF32 ? 4 : 8;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int task = blockIdx.x; task < total_tasks; task += gridDim.x) {
      TileCoord t = decode_tile(task, total_mt, n_tiles, p.num_splits, p.raster_m, s_cu_tiles, G);
      const int rows_valid = s_rows[t.g] - t.mt * kBlockM;
      const long long out_row0 = static_cast<long long>(s_row0[t.g]) + t.mt * kBlockM;
      const int col0 = t.nt * BN;
      // A k-split that owns no k-stage (more splits than stages) contributes zeros: the
      // accumulator was never written, so its contents are discarded by a zero multiplier.
      const bool empty_split = (k_stages * t.split) / p.num_splits == (k_stages * (t.split + 1)) / p.num_splits;
      const float alpha = p.group_alpha ? p.group_alpha[t.g] : 1.0f;
      if (!ptx::mbar_wait(acc_full_bar + acc, acc_phase, abort_flag, 4)) break;
      ptx::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                             static_cast<uint32_t>(acc * BN);

      auto store_chunk = [&](int chunk) {
        // staging holds 32 rows x kChunkBytes for this warp; write them out row-contiguously
        __syncwarp();
#pragma unroll
        for (int pass = 0; pass < 32 / kRowsPerPass; ++pass) {
          const int r = pass * kRowsPerPass + lane / kLanesPerRow;
          const int cc = lane % kLanesPerRow;
          const uint4 v = *reinterpret_cast<const uint4*>(my_staging + r * kStagingRowBytes + cc * 16);
          const int grow = q * 32 + r;
          const int col = col0 + chunk * kChunkCols + cc * kElemsPer16B;
          if (grow < rows_valid && col < p.n) {
            if constexpr (kOutF32) {
              float* dst = static_cast<float*>(p.out) + t.split * p.out_split_stride +
                           (out_row0 + grow) * p.n + col;
              *reinterpret_cast<uint4*>(dst) = v;
            } else {
              __half* dst = static_cast<__half*>(p.out) + t.split * p.out_split_stride +
                            (out_row0 + grow) * p.n + col;
              *reinterpret_cast<uint4*>(dst) = v;
            }
          }
        }
        __syncwarp();
      };

      if constexpr (kOutF32) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(taddr + c * 32, v);
          ptx::tmem_ld_wait();
          if (c == BN / 32 - 1) {  // accumulator fully read: hand it back to the MMA warp
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(acc_empty_bar + acc);
          }
          uint4* row = reinterpret_cast<uint4*>(my_staging + lane * kStagingRowBytes);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            uint4 o;
            o.x = empty_split ? 0u : __float_as_uint(__uint_as_float(v[4 * i + 0]) * alpha);
            o.y = empty_split ? 0u : __float_as_uint(__uint_as_float(v[4 * i + 1]) * alpha);
            o.z = empty_split ? 0u : __float_as_uint(__uint_as_float(v[4 * i + 2]) * alpha);
            o.w = empty_split ? 0u : __float_as_uint(__uint_as_float(v[4 * i + 3]) * alpha);
            row[i] = o;
          }
          store_chunk(c);
        }
      } else {
        uint32_t packed[BN / 2];
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(taddr + c * 32, v);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i)
            packed[c * 16 + i] = empty_split ? 0u
                                             : pack_half2(__uint_as_float(v[2 * i]) * alpha,
                                                          __uint_as_float(v[2 * i + 1]) * alpha);
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(acc_empty_bar + acc);
#pragma unroll
        for (int chunk = 0; chunk < BN / kChunkCols; ++chunk) {
          uint4* row = reinterpret_cast<uint4*>(my_staging + lane * kStagingRowBytes);
#pragma unroll
          for (int i = 0; i < kChunkBytes / 16; ++i) {
            const int b = chunk * (kChunkCols / 2) + 4 * i;
            row[i] = make_uint4(packed[b], packed[b + 1], packed[b + 2], packed[b + 3]);
          }
          store_chunk(chunk);
        }
      }
      if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ---- teardown
  __syncthreads();
  const int aborted = *abort_flag;
  if (aborted != 0) {
    // give copies that may still be in flight time to land before shared memory goes away
    long long start = clock64();
    while (clock64() - start < (1ll << 22)) {
    }
    if (threadIdx.x == 0 && p.error) atomicCAS(p.error, 0, aborted | (static_cast<int>(blockIdx.x) << 8));
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

}  // namespace b200
