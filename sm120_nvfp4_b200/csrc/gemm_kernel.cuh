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
// Two variants of one template:
//   one CTA per tile   128 x BN output tile, tcgen05 cta_group::1, BN = 64 / 128 / 256
//   CTA pair per tile  256 x 256 output tile computed by two CTAs of a cluster with
//                      cta_group::2 MMAs: each CTA loads its 128 rows of A and its half of
//                      B, so a pair moves 1.5x fewer operand bytes per flop than two single
//                      CTAs. No multicast load is used anywhere.
//
// Structure of one CTA (384 threads, one CTA per SM):
//   warps 0, 2, 3  loaders: one thread each issues the TMA loads of the A tile, the B tile
//                  (128-byte swizzle) and the scale-factor atoms of a k-stage into a ring of
//                  shared-memory stages; all three report to the stage's `full` barrier
//   warp 1         MMA issuer (first CTA of a pair only): per k-stage, tcgen05.cp copies the
//                  stage's scale atoms from shared into tensor memory, then tcgen05.mma
//                  kind::mxf4nvf4 (M x BN x 64 per instruction) accumulates FP32 in tensor memory;
//                  the copies and the MMAs of one thread execute in issue order, so one scale
//                  buffer in tensor memory suffices. tcgen05.commit releases the stage / publishes
//                  the tile
//   warps 4-11     epilogue: tcgen05.ld of the accumulator (a 32-lane quarter and half of the
//                  columns per warp), conversion, TMA stores through a swizzled staging buffer
//                  (ragged slabs: 16-byte stores with row / column predicates)
// Two accumulators alternate between tiles so that the epilogue of one tile overlaps the MMAs of
// the next. 256-column tiles have no room for two disjoint ones beside the scales (512 columns of
// tensor memory): theirs overlap by 64 columns, the epilogue drains those 64 first and hands them
// back early (`ovl_free`), the rest while the next tile is being computed.
// Split-K for skinny problems (kClusterSplit = 2 or 4): the CTAs of a cluster compute the same output
// tile over consecutive K ranges and reduce the FP32 partial tiles among themselves through
// distributed shared memory - each CTA collects one column slice of the tile from its peers, adds
// the partials in split order and writes that slice - so all SMs pull on the weights of a problem
// with few tiles, without a workspace, a second launch or a round trip of partial sums through HBM.
// All mbarrier waits are bounded (ptx::mbar_wait); a timeout is reported through
// GemmParams::error instead of hanging.
#pragma once

#include <cuda_fp16.h>

#include "nvfp4_math.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr int kBlockM = 128;        // rows of A per CTA = rows of one UMMA half
constexpr int kStageKBytes = 128;   // bytes of K per stage row = one swizzle span
constexpr int kStageK = 256;        // E2M1 values of K per sub-stage
constexpr int kAtomBytes = 512;     // one scale atom: 128 rows x 4 k-blocks
constexpr int kMaxGroups = 1024;
constexpr int kEpilogueWarps = 8;       // two per TMEM lane quarter, each takes half the columns
// Warp roles. Every asynchronous-copy instruction costs the issuing thread tens of
// nanoseconds, and a k-stage of FP4 MMAs lasts only ~0.3 us, so the A tile, the B tile and
// the scale atoms are each issued by a thread of their own warp.
constexpr int kWarpLoadA = 0;
constexpr int kWarpMma = 1;
constexpr int kWarpLoadB = 2;
constexpr int kWarpLoadSf = 3;
constexpr int kFirstEpilogueWarp = 4;
constexpr int kGemmThreads = 32 * (kFirstEpilogueWarp + kEpilogueWarps);
constexpr int kMaxStages = 8;
constexpr int kBarrierBytes = 256;      // 2 x kMaxStages + 7 mbarriers, TMEM base, abort flag
constexpr int kSmemBudget = 232448;     // 227 KB opt-in limit per CTA
constexpr long long kDefaultWaitLimit = 1ll << 31;   // clock cycles, about a second

// Codes a timed-out wait leaves in the device error word (low byte; the CTA index above it).
enum WaitCode { kWaitEmpty = 1, kWaitAccEmpty = 2, kWaitFull = 3, kWaitAccFull = 4, kWaitOverlap = 5,
                kWaitPartials = 7, kWaitSlots = 8 };

struct GemmParams {
  int num_groups;
  int n;                      // output columns per group
  int k;                      // logical K
  int m_uniform;              // rows per group when seqlens == nullptr
  const int* seqlens;         // [G] valid rows per group (device) or nullptr
  const int* cu_seqlens;      // [G+1] first row of each group (device) or nullptr
  int sfa_group_atom_rows;    // 128-row atom rows in one group's SFA region
  int sfb_group_atom_rows;    // ... in one group's SFB region (0 when every group shares one B)
  int b_group_rows;           // rows of B per group (N), 0 when every group shares one B
  void* out;                  // FP16 or FP32 [rows, n]
  long long out_split_stride;  // elements between split-K slices of `out`
  const float* group_alpha;   // optional per-group multiplier applied in FP32
  int num_splits;             // split-K factor (1 = none)
  int raster_m;               // m-tiles per rasterisation band
  int* tiles_out;             // optional [G]   ceil(rows/128) per group
  int* cu_tiles_out;          // optional [G+1] exclusive prefix of tiles_out
  int* error;                 // device word that receives a non-zero code on a timed-out wait
  int a_sub_bytes;            // shared-memory bytes of one sub-stage of A: rows in the A box x 128
  int num_stages;             // depth of the operand ring in shared memory (<= kMaxStages)
  long long out_ld;           // elements between output rows (n, or the full width when n is a column window)
  int tma_store;              // 1: the output tensor map is valid, full 32-row slabs go out by TMA store
  int out_rows_per_split;     // rows between split-K slices in the output tensor map (M), 0 without split
  // Fused gate/up variant (kSwiGlu kernels): B holds [gate rows 0..I) ; up rows I..2I) per group, a
  // tile computes 128 gate and the matching 128 up columns, and the epilogue writes
  // NVFP4(silu(gate) * up) instead of the FP16 product.
  int swiglu_inter;           // I (multiple of 128), 0 for plain GEMMs
  uint8_t* q_out;             // packed E2M1 [rows, I/2]
  uint8_t* q_scale;           // UE4M3 scale regions, one per group, indexed by the row inside the group
  long long q_scale_group_stride;
  int red_bytes;              // cluster split-K: bytes of the partial-tile slots in shared memory, else 0
  long long wait_limit;       // clock cycles a wait may last (kDefaultWaitLimit)
  int withhold_first_arrival;  // test hook: the scale loader of CTA 0 skips its first arrival, so the
                               // first k-stage never becomes ready and the waits run out
};

template <int BN, bool kTwoCta>
struct GemmCfg {
  // Tiles narrower than 128 columns select their part of a 128-row scale atom by offsetting
  // the TMEM address of the scale columns; the hardware wants that address two-column
  // aligned, which rules out 32-wide tiles (they would need odd offsets).
  static_assert(BN == 64 || BN == 128 || BN == 256, "unsupported tile width");
  static_assert(!kTwoCta || BN == 256, "the CTA-pair variant is built for 256-wide tiles");
  static constexpr int kCtas = kTwoCta ? 2 : 1;
  static constexpr int kTileM = kBlockM * kCtas;            // rows of one output tile
  static constexpr int kBRows = BN / kCtas;                 // rows of B this CTA loads
  static constexpr int kSfbGroups = (BN + 127) / 128;       // 128-row scale tiles per B tile
  static constexpr int kSfbColsPerMma = 4 * kSfbGroups;     // TMEM columns of SFB per MMA
  // Sub-stages per pipeline stage. One sub-stage is 256 k-values (one 128-byte swizzle span, four
  // MMAs). A barrier round - waits, arrivals, commit - costs several hundred cycles whatever it
  // carries; for 64-column tiles (skinny problems, bound by streaming B) two sub-stages per round
  // halve the rounds per byte.
  static constexpr int kSub = BN == 64 ? 2 : 1;
  static constexpr int kAtomsPerStage = 4 * kSub;
  // Tensor memory: two accumulators, then the scale columns of one k-stage (SFA 4 per MMA, SFB
  // BN / 32 per MMA). 256-column accumulators overlap by 64 columns (see the file header).
  static constexpr bool kOverlap = BN == 256;
  static constexpr int kAccStride = kOverlap ? 192 : BN;
  static constexpr int kSfBase = kAccStride + BN;
  static constexpr int kSfColsPerSub = 16 + 4 * kSfbColsPerMma;   // 4 MMAs: SFA 4x4, SFB 4xN/32
  static constexpr int kSfCols = kSub * kSfColsPerSub;
  static constexpr int kTmemCols = kSfBase + kSfCols <= 256 ? 256 : 512;
  static_assert(kSfBase + kSfCols <= 512, "tensor memory overcommitted");
  static_assert(!kOverlap || BN - kAccStride == 64, "the epilogue drains a 64-column overlap first");
  // One sub-stage of A: 128 rows, or fewer when the whole problem has fewer rows (the loader's box
  // then covers round-up-to-8 rows; the MMA still reads 128 rows' worth of shared memory, the rest
  // being whatever follows - rows that are never stored). The freed space deepens the ring, which
  // is what a skinny problem needs: it is bound by the bytes of B in flight.
  static constexpr int kABytes = kBlockM * kStageKBytes;
  static constexpr int kBBytes = kBRows * kStageKBytes;            // one sub-stage of B
  static constexpr int kSfaBytes = 4 * kAtomBytes;                 // one sub-stage of SFA atoms
  static constexpr int kSfbBytes = kSfbGroups * 4 * kAtomBytes;
  // stage layout: [A sub-stages][B sub-stages][SFA atoms][SFB atoms of scale tile 0][scale tile 1]
  __host__ __device__ static constexpr int stage_bytes(int a_sub_bytes) {
    return kSub * (a_sub_bytes + kBBytes + kSfaBytes + kSfbBytes);
  }
  // Output staging for TMA stores: 32 rows x 128 bytes per epilogue warp. Tiles of 64 columns
  // give a warp only 32 columns (64 bytes of FP16 per row) and keep the direct-store epilogue.
  static constexpr int kStagingWarpBytes = 32 * 128;
  static constexpr int kStagingBytes = BN >= 128 ? kEpilogueWarps * kStagingWarpBytes : 0;

  // Shared memory: [operand stages][output staging][barriers][group tables]; +1024 slack to align the base.
  static constexpr int fixed_bytes(int num_groups) {
    return 1024 + kBarrierBytes + 3 * (num_groups + 1) * 4 + kStagingBytes;
  }
  // Cluster split-K: a CTA keeps one slot of 128 rows x BN / splits FP32 columns per peer.
  static constexpr int red_bytes(int splits) { return splits > 1 ? (splits - 1) * kBlockM * (BN / splits) * 4 : 0; }
  static constexpr int stages_for(int num_groups, int a_sub_bytes = kABytes, int extra_bytes = 0) {
    // the MMA reads a full 128-row A block from the last sub-stage, so that much shared memory
    // must follow it: B, the scales and the staging area do
    int s = (kSmemBudget - fixed_bytes(num_groups) - extra_bytes) / stage_bytes(a_sub_bytes);
    return s > kMaxStages ? kMaxStages : s;
  }
  static constexpr int smem_bytes(int num_groups, int a_sub_bytes = kABytes, int extra_bytes = 0) {
    return fixed_bytes(num_groups) + extra_bytes +
           stages_for(num_groups, a_sub_bytes, extra_bytes) * stage_bytes(a_sub_bytes);
  }
  static_assert(stages_for(kMaxGroups) >= 3, "pipeline too shallow");
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

template <int BN, bool kOutF32, bool kTwoCta, bool kSwiGlu = false, int kClusterSplit = 1>
__global__ void __launch_bounds__(kGemmThreads, 1)
nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                  const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_out,
                  const __grid_constant__ CUtensorMap tmap_sfa,
                  const __grid_constant__ CUtensorMap tmap_sfb, const GemmParams p) {
  using Cfg = GemmCfg<BN, kTwoCta>;
  static_assert(!kSwiGlu || (BN == 256 && !kOutF32), "the fused gate/up epilogue is built on 256-column FP16 tiles");
  static_assert(kClusterSplit == 1 || (!kTwoCta && !kSwiGlu && !kOutF32 && BN <= 128 &&
                                       (kClusterSplit == 2 || kClusterSplit == 4)),
                "cluster split-K: single-CTA FP16 tiles of 64 or 128 columns, 2 or 4 splits");
  constexpr bool kSplitCluster = kClusterSplit > 1;
  constexpr int kCtas = Cfg::kCtas;
  constexpr int kTileM = Cfg::kTileM;
  constexpr int kSub = Cfg::kSub;
  constexpr int kAtomsPerStage = Cfg::kAtomsPerStage;
  constexpr bool kOverlap = Cfg::kOverlap;
  const int kStages = p.num_stages;
  const long long wait_limit = p.wait_limit;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t a_bytes = static_cast<uint32_t>(p.a_sub_bytes);
  const uint32_t stage_bytes = static_cast<uint32_t>(Cfg::stage_bytes(p.a_sub_bytes));
  uint8_t* staging_base = smem + kStages * stage_bytes;   // 1024-byte aligned: stages are multiples of 1 KB
  // full:      the stage is ready for the MMAs: its A / B tiles and its scale atoms landed in shared
  //            memory (pair: in both CTAs; the barrier lives in the first CTA)
  // empty:     the copies and MMAs that read the stage are done
  // acc_full:  an accumulator holds a finished tile          acc_empty: the epilogue has read all of it
  // ovl_free:  (overlapping accumulators) the epilogue has read the 64 columns the other accumulator shares
  // red_full:  (cluster split-K) every peer has stored its partial of this CTA's column slice
  // red_empty: (cluster split-K) every peer has read the partials this CTA stored into it
  uint8_t* red_base = staging_base + Cfg::kStagingBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(red_base + p.red_bytes);
  const uint32_t full_u32 = ptx::smem_u32(bars);
  const uint32_t empty_u32 = full_u32 + 8 * kMaxStages;
  const uint32_t acc_full_u32 = empty_u32 + 8 * kMaxStages;
  const uint32_t acc_empty_u32 = acc_full_u32 + 16;
  const uint32_t ovl_free_u32 = acc_empty_u32 + 16;
  const uint32_t red_full_u32 = ovl_free_u32 + 8;
  const uint32_t red_empty_u32 = red_full_u32 + 8;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 7);
  int* abort_flag = reinterpret_cast<int*>(tmem_holder + 1);
  int* s_cu_tiles = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + kBarrierBytes);
  int* s_row0 = s_cu_tiles + (p.num_groups + 1);
  int* s_rows = s_row0 + (p.num_groups + 1);

  // The warp index comes out of a shuffle so that the compiler can prove it uniform across the
  // warp: the role branches below then are uniform branches, and the barrier addresses, ring
  // positions and descriptors inside them stay in uniform registers instead of being moved
  // there from vector registers for every mbarrier / TMA / tcgen05 instruction.
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const int G = p.num_groups;
  const uint32_t cta_rank = kTwoCta ? ptx::cluster_cta_rank() : 0u;
  const bool leader = cta_rank == 0;
  const int split_rank = kSplitCluster ? static_cast<int>(ptx::cluster_cta_rank()) : 0;   // this CTA's K range
  constexpr int kClusterCtas = kCtas * kClusterSplit;
  const int worker = static_cast<int>(blockIdx.x) / kClusterCtas;     // CTA, CTA pair or split-K cluster
  const int num_workers = static_cast<int>(gridDim.x) / kClusterCtas;
  const int num_splits = kSplitCluster ? kClusterSplit : p.num_splits;   // K ranges per tile
  const int task_splits = kSplitCluster ? 1 : p.num_splits;              // ... that are tasks of their own

  // every warp that will use a tensor map fetches its descriptor now, in parallel with the set-up
  if (lane == 0) {
    if (warp == kWarpLoadA) ptx::prefetch_tensormap(&tmap_a);
    if (warp == kWarpLoadB) ptx::prefetch_tensormap(&tmap_b);
    if (warp == kWarpLoadSf) { ptx::prefetch_tensormap(&tmap_sfa); ptx::prefetch_tensormap(&tmap_sfb); }
    if (warp == kFirstEpilogueWarp && p.tma_store) ptx::prefetch_tensormap(&tmap_out);
  }
  // ---- group tables: valid rows, first row and m-tile prefix of every group
  for (int g = threadIdx.x; g < G; g += kGemmThreads) {
    int rows = p.seqlens ? p.seqlens[g] : p.m_uniform;
    rows = rows > 0 ? rows : 0;
    s_rows[g] = rows;
    s_row0[g] = p.cu_seqlens ? p.cu_seqlens[g] : g * p.m_uniform;
    s_cu_tiles[g] = (rows + kTileM - 1) / kTileM;
  }
  // Set-up runs in parallel: the lanes of warp 0 initialise one barrier each, the MMA warp
  // allocates tensor memory meanwhile. A single problem (one group) needs no scan of tile counts;
  // its loaders start as soon as the barriers exist, without waiting for the tensor-memory
  // allocation (`fast_start`): on a skinny problem the first bytes from HBM are the critical path.
  const bool fast_start = !kTwoCta && G == 1;
  if (G == 1 && threadIdx.x == 0) {   // this thread wrote the only table entry itself
    const int tiles = s_cu_tiles[0];
    s_cu_tiles[0] = 0;
    s_cu_tiles[1] = tiles;
    if (blockIdx.x == 0) {
      const int t128 = (s_rows[0] + kBlockM - 1) / kBlockM;
      if (p.tiles_out) p.tiles_out[0] = t128;
      if (p.cu_tiles_out) { p.cu_tiles_out[0] = 0; p.cu_tiles_out[1] = t128; }
    }
  }
  if (warp == 0) {
    if (lane == 0) *abort_flag = 0;
    for (int s = lane; s < kStages; s += 32) {
      ptx::mbar_init(full_u32 + 8 * s, 3);     // the A, the B and the scale loader of the owning CTA
      ptx::mbar_init(empty_u32 + 8 * s, 1);
    }
    if (lane < 2) {
      ptx::mbar_init(acc_full_u32 + 8 * lane, 1);
      ptx::mbar_init(acc_empty_u32 + 8 * lane, kEpilogueWarps * kCtas);
    }
    if (lane == 2) ptx::mbar_init(ovl_free_u32, (kEpilogueWarps / 2) * kCtas);
    if (lane == 3) ptx::mbar_init(red_full_u32, 1);     // the announcing thread; the partials arrive as counted bytes
    if (lane == 4) ptx::mbar_init(red_empty_u32, kEpilogueWarps * (kClusterSplit - 1) + (kSplitCluster ? 0 : 1));
    __syncwarp();
    if (lane == 0) ptx::fence_barrier_init();
  }
  const bool loader_warp = warp == kWarpLoadA || warp == kWarpLoadB || warp == kWarpLoadSf;
  if (fast_start) {
    // Two named barriers over the whole CTA. 1 = "barriers and tables exist": everybody arrives, only
    // the loaders wait for it. 2 = "tensor memory allocated": everybody arrives (the loaders at once),
    // the MMA and epilogue warps wait.
    if (loader_warp) {
      ptx::named_barrier_sync(1, kGemmThreads);
      ptx::named_barrier_arrive(2, kGemmThreads);
    } else {
      ptx::named_barrier_arrive(1, kGemmThreads);
      if (warp == kWarpMma) {
        ptx::tmem_alloc<kCtas>(ptx::smem_u32(tmem_holder), Cfg::kTmemCols);
        ptx::tmem_relinquish<kCtas>();
      }
      ptx::tc_fence_before_sync();
      ptx::named_barrier_sync(2, kGemmThreads);
    }
  } else if (warp == kWarpMma) {
    ptx::tmem_alloc<kCtas>(ptx::smem_u32(tmem_holder), Cfg::kTmemCols);
    ptx::tmem_relinquish<kCtas>();
  }
  if (G > 1) {
    __syncthreads();
    if (warp == kWarpLoadA) {  // exclusive scan of the per-group tile counts, 32 groups at a time
      int carry = 0;
      for (int base = 0; base < G; base += 32) {
        int v = (base + lane < G) ? s_cu_tiles[base + lane] : 0;
        int incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          int o = __shfl_up_sync(0xffffffffu, incl, d);
          if (lane >= d) incl += o;
        }
        if (base + lane < G) s_cu_tiles[base + lane] = carry + incl - v;
        carry += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) s_cu_tiles[G] = carry;
      if (blockIdx.x == 0 && (p.tiles_out || p.cu_tiles_out)) {
        // the reference ABI's scratch outputs: 128-row tile count per group and its prefix
        int run = 0;
        for (int base = 0; base < G; base += 32) {
          int v = (base + lane < G) ? (s_rows[base + lane] + kBlockM - 1) / kBlockM : 0;
          int incl = v;
#pragma unroll
          for (int d = 1; d < 32; d <<= 1) {
            int o = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += o;
          }
          if (base + lane < G) {
            if (p.tiles_out) p.tiles_out[base + lane] = v;
            if (p.cu_tiles_out) p.cu_tiles_out[base + lane] = run + incl - v;
          }
          run += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0 && p.cu_tiles_out) p.cu_tiles_out[G] = run;
      }
    }
  }
  if (!fast_start) {
    ptx::tc_fence_before_sync();
    __syncthreads();
  }
  // The partners' barriers must exist before anything is signalled to them. A pair does so from its
  // first load on; a split-K cluster only in its epilogues, so its threads just announce themselves
  // here and wait for the others where they first need them.
  if constexpr (kTwoCta) {
    ptx::cluster_arrive_relaxed();
    ptx::cluster_wait();
  }
  if constexpr (kSplitCluster) ptx::cluster_arrive_relaxed();
  ptx::tc_fence_after_sync();

  const uint32_t tmem_base = *tmem_holder;
  const int total_mt = s_cu_tiles[G];
  // fused gate/up: a tile covers 128 columns of the intermediate (its gate and its up half)
  const int n_tiles = kSwiGlu ? p.swiglu_inter / 128 : (p.n + BN - 1) / BN;
  const int total_tasks = total_mt * n_tiles * task_splits;
  const int kt = (p.k + 63) / 64;               // scale atoms along K
  const int k_stages = (kt + kAtomsPerStage - 1) / kAtomsPerStage;   // pipeline stages along K
  const int k_stages_full = kt / kAtomsPerStage;                     // k-stages with all their atoms

  // 32-bit shared-window addresses of the ring: the role loops below advance them with adds.
  const uint32_t stage_u32 = ptx::smem_u32(smem);
  // where completion bytes for a stage's `full` barrier go: this CTA's barrier, or the first CTA's
  const uint32_t full_target_u32 = kTwoCta ? ptx::map_to_cta(full_u32, 0) : full_u32;
  // offsets inside a stage
  const uint32_t off_b = kSub * a_bytes;
  const uint32_t off_sfa = off_b + kSub * Cfg::kBBytes;
  const uint32_t off_sfb = off_sfa + kSub * Cfg::kSfaBytes;

  if (warp == kWarpLoadA || warp == kWarpLoadB || warp == kWarpLoadSf) {
    // ================================ loaders ================================
    // One thread per operand class. Completion bytes are counted on the barrier of the first CTA
    // (in a pair both CTAs' loads report there, and only the first CTA's loaders arm it, for both
    // halves), so the MMA issuer waits on one barrier per stage. Boxes that reach past the end of
    // a matrix (K tail, last rows) are completed with zeros by the copy engine and still count
    // their full size.
    const int role = warp == kWarpLoadA ? 0 : (warp == kWarpLoadB ? 1 : 2);
    const uint32_t role_bytes =
        role == 0 ? kSub * a_bytes
                  : (role == 1 ? static_cast<uint32_t>(kSub * Cfg::kBBytes)
                               : static_cast<uint32_t>(kSub * (Cfg::kSfaBytes + Cfg::kSfbBytes)));
    int stage = 0;
    uint32_t phase = 0, dst = stage_u32, full_a = full_u32, full_t = full_target_u32, empty_a = empty_u32;
    bool withhold = role == 2 && p.withhold_first_arrival != 0 && blockIdx.x == 0;
    bool ok = true;
    for (int task = worker; task < total_tasks && ok; task += num_workers) {
      TileCoord t = decode_tile(task, total_mt, n_tiles, task_splits, p.raster_m, s_cu_tiles, G);
      if constexpr (kSplitCluster) t.split = split_rank;
      int row = 0, row2 = 0;   // A / B: matrix row of the box; scales: atom rows of SFA and SFB
      if (role == 0) {
        row = s_row0[t.g] + t.mt * kTileM + static_cast<int>(cta_rank) * kBlockM;
      } else if (role == 1) {
        if constexpr (kSwiGlu) row = t.g * p.b_group_rows + t.nt * 128 + (kTwoCta ? static_cast<int>(cta_rank) * p.swiglu_inter : 0);
        else row = t.g * p.b_group_rows + t.nt * BN + static_cast<int>(cta_rank) * Cfg::kBRows;
      } else {
        row = t.g * p.sfa_group_atom_rows + t.mt * kCtas + static_cast<int>(cta_rank);
        row2 = t.g * p.sfb_group_atom_rows + (kSwiGlu ? t.nt : (t.nt * BN) / 128);
      }
      const int ks_begin = (k_stages * t.split) / num_splits;
      const int ks_end = (k_stages * (t.split + 1)) / num_splits;
      for (int ks = ks_begin; ks < ks_end; ++ks) {
        if (!ptx::mbar_wait(empty_a, phase ^ 1, abort_flag, kWaitEmpty, wait_limit)) { ok = false; break; }
        if (ptx::elect_one()) {
          if (withhold) {
            withhold = false;
          } else if (!kTwoCta || leader) {
            ptx::mbar_arrive_expect_tx(full_a, kCtas * role_bytes);
          }
          if (role == 2) {
            const int atom0 = ks * kAtomsPerStage;
            if constexpr (kTwoCta) {
              ptx::tma_load_3d_pair(dst + off_sfa, &tmap_sfa, full_t, 0, atom0, row);
              if constexpr (kSwiGlu) {
                ptx::tma_load_3d_pair(dst + off_sfb, &tmap_sfb, full_t, 0, atom0, row2);
                ptx::tma_load_3d_pair(dst + off_sfb + kAtomsPerStage * kAtomBytes, &tmap_sfb, full_t, 0, atom0,
                                      row2 + p.swiglu_inter / 128);
              } else {
                ptx::tma_load_3d_pair(dst + off_sfb, &tmap_sfb, full_t, 0, atom0, row2);
              }
            } else {
              ptx::tma_load_3d(dst + off_sfa, &tmap_sfa, full_a, 0, atom0, row);
              if constexpr (kSwiGlu) {
                ptx::tma_load_3d(dst + off_sfb, &tmap_sfb, full_a, 0, atom0, row2);
                ptx::tma_load_3d(dst + off_sfb + kAtomsPerStage * kAtomBytes, &tmap_sfb, full_a, 0, atom0,
                                 row2 + p.swiglu_inter / 128);
              } else {
                ptx::tma_load_3d(dst + off_sfb, &tmap_sfb, full_a, 0, atom0, row2);
              }
            }
          } else {
            const CUtensorMap* tmap = role == 0 ? &tmap_a : &tmap_b;
            const uint32_t sub_bytes = role == 0 ? a_bytes : static_cast<uint32_t>(Cfg::kBBytes);
            const uint32_t d0 = dst + (role == 0 ? 0u : off_b);
            const int c0 = ks * kSub * kStageKBytes;
            if constexpr (kTwoCta) {
#pragma unroll
              for (int sub = 0; sub < kSub; ++sub)
                ptx::tma_load_2d_pair(d0 + sub * sub_bytes, tmap, full_t, c0 + sub * kStageKBytes, row);
            } else if (kSwiGlu && role == 1) {   // 128 gate rows, then the 128 up rows I further down (128-row box)
              ptx::tma_load_2d(d0, tmap, full_a, c0, row);
              ptx::tma_load_2d(d0 + sub_bytes / 2, tmap, full_a, c0, row + p.swiglu_inter);
            } else {
#pragma unroll
              for (int sub = 0; sub < kSub; ++sub)
                ptx::tma_load_2d(d0 + sub * sub_bytes, tmap, full_a, c0 + sub * kStageKBytes, row);
            }
          }
        }
        dst += stage_bytes; full_a += 8; full_t += 8; empty_a += 8;
        if (++stage == kStages) {
          stage = 0; phase ^= 1; dst = stage_u32; full_a = full_u32; full_t = full_target_u32; empty_a = empty_u32;
        }
      }
    }
    __syncwarp();
  } else if (warp == kWarpMma) {
    // =============================== MMA issuer ==============================
    if (leader) {
      constexpr uint32_t idesc = ptx::make_idesc_nvfp4(kTileM, BN);
      constexpr uint16_t kAllCtas = kTwoCta ? 3 : 1;
      const uint32_t kDescStep = stage_bytes >> 4;                 // descriptor units per stage
      const uint32_t a_desc_sub = a_bytes >> 4;                    // ... per sub-stage of A
      const uint32_t a_lo0 = ptx::kmajor_sw128_desc_lo(stage_u32);
      const uint32_t sf_col = tmem_base + Cfg::kSfBase;
      int stage = 0, acc = 0, tile_iter = 0;
      uint32_t phase = 0, acc_phase = 0, full_a = full_u32, empty_a = empty_u32, a_lo = a_lo0;
      bool ok = true;
      for (int task = worker; task < total_tasks && ok; task += num_workers, ++tile_iter) {
        TileCoord t = decode_tile(task, total_mt, n_tiles, task_splits, p.raster_m, s_cu_tiles, G);
      if constexpr (kSplitCluster) t.split = split_rank;
        const int ks_begin = (k_stages * t.split) / num_splits;
        const int ks_end = (k_stages * (t.split + 1)) / num_splits;
        // A tile narrower than 128 columns uses part of a 128-row scale atom: column
        // (n0 % 128) / 32 of the four TMEM columns the atom occupies.
        const uint32_t sfb_sub = BN < 128 ? static_cast<uint32_t>(((t.nt * BN) % 128) / 32) : 0u;
        // this accumulator's previous tile has been read completely ...
        if (!ptx::mbar_wait(acc_empty_u32 + 8 * acc, acc_phase ^ 1, abort_flag, kWaitAccEmpty, wait_limit)) break;
        // ... and the previous tile (in the other accumulator) no longer needs the shared columns
        if (kOverlap && tile_iter > 0 &&
            !ptx::mbar_wait(ovl_free_u32, static_cast<uint32_t>(tile_iter - 1) & 1u, abort_flag, kWaitOverlap, wait_limit))
          break;
        ptx::tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(acc * Cfg::kAccStride);
        // The tensor pipe accepts an MMA only when the previous one is almost done (issuing
        // four 128-cycle MMAs occupies this thread for 512 cycles), so whatever this thread does
        // between the last MMA of a k-stage and the first of the next must fit into one MMA's
        // run time or the pipe idles. The next stage's barrier is therefore probed between the
        // third and the fourth MMA, while the pipe is busy.
        bool ready = false;
        for (int ks = ks_begin; ks < ks_end; ++ks) {
          if (!ready && !ptx::mbar_wait(full_a, phase, abort_flag, kWaitFull, wait_limit)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t b_lo = a_lo + (off_b >> 4);
          // scale-atom descriptors: the same 16-byte address field, no leading-dimension offset
          const uint32_t sfa_lo = a_lo - ptx::kKmajorSw128LboBits + (off_sfa >> 4);
          const uint32_t sfb_lo = a_lo - ptx::kKmajorSw128LboBits + (off_sfb >> 4);
          const bool last_ring = stage + 1 == kStages;
          const uint32_t next_full = last_ring ? full_u32 : full_a + 8;
          const uint32_t next_phase = last_ring ? phase ^ 1 : phase;
          // Scale atoms of the stage: shared -> tensor memory. Atom (sub, j) of SFA goes to the four
          // columns MMA j of sub-stage `sub` reads; atom (gi, sub, j) of SFB to columns 4 gi.. of that MMA.
          auto copy_scales = [&](int atoms) {
#pragma unroll
            for (int i = 0; i < kAtomsPerStage; ++i) {
              if (i < atoms) {
                const int sub = i >> 2, j = i & 3;
                const uint32_t col = sf_col + sub * Cfg::kSfColsPerSub;
                ptx::tc_cp_32x128b_warpx4<kCtas>(col + 4 * j, sfa_lo + i * (kAtomBytes >> 4),
                                                 ptx::kSfAtomDescHi);
#pragma unroll
                for (int gi = 0; gi < Cfg::kSfbGroups; ++gi)
                  ptx::tc_cp_32x128b_warpx4<kCtas>(col + 16 + j * Cfg::kSfbColsPerMma + 4 * gi,
                                                   sfb_lo + (gi * kAtomsPerStage + i) * (kAtomBytes >> 4),
                                                   ptx::kSfAtomDescHi);
              }
            }
          };
          // MMA number i of the stage (sub-stage i / 4, atom i % 4): 64 E2M1 values = 32 bytes along K
          // are +2 in the descriptor's 16-byte address field; a sub-stage is one operand block further
          auto issue = [&](int i, uint32_t accumulate) {
            const int sub = i >> 2, j = i & 3;
            const uint32_t col = sf_col + sub * Cfg::kSfColsPerSub;
            ptx::tc_mma_nvfp4<kCtas>(tmem_acc, a_lo + sub * a_desc_sub + 2 * j,
                                     b_lo + sub * (Cfg::kBBytes >> 4) + 2 * j, ptx::kKmajorSw128DescHi, idesc,
                                     col + 4 * j, col + 16 + j * Cfg::kSfbColsPerMma + sfb_sub, accumulate);
          };
          if (ks < k_stages_full) {
            if (ptx::elect_one()) {
              copy_scales(kAtomsPerStage);
              issue(0, ks > ks_begin ? 1u : 0u);
#pragma unroll
              for (int i = 1; i < kAtomsPerStage - 1; ++i) issue(i, 1u);
            }
            ready = ks + 1 < ks_end && __all_sync(0xffffffffu, ptx::mbar_test_wait(next_full, next_phase));
            if (ptx::elect_one()) {
              issue(kAtomsPerStage - 1, 1u);
              ptx::tc_commit<kCtas>(empty_a, kAllCtas);
            }
          } else {
            ready = false;
            if (ptx::elect_one()) {
              const int atoms = kt - ks * kAtomsPerStage;    // K tail: fewer atoms than a stage holds
              copy_scales(atoms);
              for (int i = 0; i < atoms && i < kAtomsPerStage; ++i) issue(i, (i > 0 || ks > ks_begin) ? 1u : 0u);
              ptx::tc_commit<kCtas>(empty_a, kAllCtas);
            }
          }
          full_a += 8; empty_a += 8; a_lo += kDescStep;
          if (++stage == kStages) { stage = 0; phase ^= 1; full_a = full_u32; empty_a = empty_u32; a_lo = a_lo0; }
        }
        if (!ok) break;
        if (ptx::elect_one()) ptx::tc_commit<kCtas>(acc_full_u32 + 8 * acc, kAllCtas);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
    __syncwarp();
  } else {
    // ================================ epilogue ===============================
    // Warp w reads TMEM lanes 32*(w%4).. (a hardware rule) and half of the tile's columns;
    // each thread holds one output row of the warp's 32-row slab.
    //   * A slab whose 32 rows are all valid leaves through shared memory: every lane writes
    //     128 bytes of its row into the warp's staging buffer (128-byte swizzle, conflict-free),
    //     one lane issues a TMA store of the 32 x 128-byte box. The store engine writes whole
    //     lines; the load/store pipe sees 8 shared-memory stores per lane instead of row-strided
    //     global stores that would occupy it for thousands of cycles per tile and hold up every
    //     mbarrier operation of the other warps on the SM.
    //   * A ragged slab (end of a group, end of the matrix) and 64-column tiles use predicated
    //     16-byte global stores.
    const int q = warp & 3;
    const int half = (warp - kFirstEpilogueWarp) >> 2;
    constexpr int kWarpCols = BN / 2;                                 // columns per warp
    constexpr int kLdCols = 32;                                       // columns per TMEM load
    constexpr bool kCanStage = Cfg::kStagingBytes > 0;
    const uint32_t stg = ptx::smem_u32(staging_base) + (warp - kFirstEpilogueWarp) * Cfg::kStagingWarpBytes;
    const uint32_t stg_row = stg + lane * 128;
    int acc = 0, tile_iter = 0;
    uint32_t acc_phase = 0;
    if constexpr (kSplitCluster) ptx::cluster_wait();     // every CTA of the cluster has initialised its barriers
    for (int task = worker; task < total_tasks; task += num_workers, ++tile_iter) {
      TileCoord t = decode_tile(task, total_mt, n_tiles, task_splits, p.raster_m, s_cu_tiles, G);
      if constexpr (kSplitCluster) t.split = split_rank;
      const int slab_row = static_cast<int>(cta_rank) * kBlockM + q * 32;   // first row of the slab in the tile
      const int row_in_tile = slab_row + lane;
      const bool row_ok = t.mt * kTileM + row_in_tile < s_rows[t.g];
      const bool slab_full = t.mt * kTileM + slab_row + 32 <= s_rows[t.g];
      const long long out_row = static_cast<long long>(s_row0[t.g]) + t.mt * kTileM + row_in_tile;
      const int col0 = t.nt * BN + half * kWarpCols;
      // A k-split that owns no k-stage (more splits than stages) contributes zeros: the
      // accumulator was never written, so its contents are replaced, not scaled.
      const bool empty_split = (k_stages * t.split) / num_splits == (k_stages * (t.split + 1)) / num_splits;
      const float alpha = p.group_alpha ? p.group_alpha[t.g] : 1.0f;
      const bool staged = kCanStage && p.tma_store != 0 && slab_full;
      // row coordinate of the slab in the output tensor map (split-K slices are stacked)
      const int map_row = s_row0[t.g] + t.mt * kTileM + slab_row + t.split * p.out_rows_per_split;
      // Overlapping accumulators: accumulator 0 shares its last 64 columns with accumulator 1's first
      // 64. Those belong to the second column half of a tile in accumulator 0 and to the first half of
      // a tile in accumulator 1; the warps that hold them read them first and report on `ovl_free`.
      const bool ovl_mine = kOverlap && (acc == 0) == (half == 1);
      const bool reversed = kOverlap && acc == 0;     // read this warp's columns from the top down
      if (!ptx::mbar_wait(acc_full_u32 + 8 * acc, acc_phase, abort_flag, kWaitAccFull, wait_limit)) break;
      ptx::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                             static_cast<uint32_t>(acc * Cfg::kAccStride + half * kWarpCols);
      auto arrive_leader = [&](uint32_t bar) {   // one arrival per warp on a barrier of the first CTA
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (kTwoCta && !leader) ptx::mbar_arrive_cluster(ptx::map_to_cta(bar, 0));
          else ptx::mbar_arrive(bar);
        }
      };
      auto release_overlap = [&]() { if (ovl_mine) arrive_leader(ovl_free_u32); };
      auto release_accumulator = [&]() { arrive_leader(acc_empty_u32 + 8 * acc); };   // accumulator fully read
      // Staged output of 128 bytes per lane (eight 16-byte units in w[0..31]) in two steps, so
      // that the accumulator can be released between them: fill the warp's staging buffer, then
      // hand the 32 x 128-byte box at column `col` to the store engine.
      auto wait_staging_free = [&]() {   // the previous box has left the buffer
        if (lane == 0) ptx::bulk_wait_group_read<0>();
        __syncwarp();
      };
      auto fill_staging = [&](const uint32_t* w) {
#pragma unroll
        for (int u = 0; u < 8; ++u)
          ptx::st_shared_v4(stg_row + (static_cast<uint32_t>(u ^ (lane & 7)) << 4), w[4 * u], w[4 * u + 1],
                            w[4 * u + 2], w[4 * u + 3]);
        ptx::fence_proxy_async_smem();
      };
      auto store_staging = [&](int col) {
        __syncwarp();
        if (lane == 0) {
          ptx::tma_store_2d(&tmap_out, stg, col, map_row);
          ptx::bulk_commit_group();
        }
      };

      if constexpr (kSplitCluster) {
        // Cluster split-K. This CTA holds the partial tile of K range `me`; CTA d of the cluster finishes
        // columns [d W, (d + 1) W) of the tile. Every warp (32 rows, half of each slice's columns):
        //   1. stores its part of the other CTAs' slices into their shared memory (one slot per sender;
        //      16-byte units, swizzled by row) with asynchronous stores that count their bytes on the
        //      receiver's `red_full` barrier;
        //   2. keeps its part of this CTA's own slice in registers and hands the accumulator back;
        //   3. waits for the peers' partials, adds all of them in split order 0 .. S-1 in FP32 (the order
        //      of the reference's split-K reduction, src/gemm/specialized/m128_gemm.cu:367-382), rounds
        //      once to FP16 and stores;
        //   4. tells the peers that their slots may be overwritten (`red_empty`).
        constexpr int S = kClusterSplit, W = BN / S, HW = W / 2, kRowChunks = W / 4;
        constexpr uint32_t kSlotBytes = kBlockM * W * 4;
        const uint32_t red_u32 = ptx::smem_u32(red_base);
        const int me = split_rank;
        const int trow = q * 32 + lane;                          // row of the tile this lane holds
        const uint32_t row_off = static_cast<uint32_t>(trow) * (W * 4);
        const uint32_t swz = static_cast<uint32_t>(trow & (kRowChunks - 1) & 7);
        const uint32_t acc_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                  static_cast<uint32_t>(acc * Cfg::kAccStride + half * HW);
        if (tile_iter > 0 && !ptx::mbar_wait_cluster(red_empty_u32, static_cast<uint32_t>(tile_iter - 1) & 1u,
                                                     abort_flag, kWaitSlots, wait_limit))
          break;
        // One thread announces what this CTA is about to receive: every peer sends the valid rows of
        // this CTA's slice, 4 W bytes per row, as asynchronous stores that report their bytes to
        // `red_full` themselves - no fence and no separate signal on the sending side.
        const int rows_here = min(kBlockM, s_rows[t.g] - t.mt * kTileM);
        if (warp == kFirstEpilogueWarp && lane == 0)
          ptx::mbar_arrive_expect_tx(red_full_u32, static_cast<uint32_t>((S - 1) * rows_here * W * 4));
        // all partial slices for the peers first (one wait for the loads), then the stores
        uint32_t snd[S - 1][HW];
#pragma unroll
        for (int dd = 1; dd < S; ++dd) {
          const int d = (me + dd) % S;
#pragma unroll
          for (int c8 = 0; c8 < HW / 8; ++c8) ptx::tmem_ld_32x32b_x8(acc_addr + d * W + c8 * 8, &snd[dd - 1][c8 * 8]);
        }
        ptx::tmem_ld_wait();
#pragma unroll
        for (int dd = 1; dd < S; ++dd) {
          const int d = (me + dd) % S;
          const uint32_t remote = ptx::map_to_cta(red_u32 + static_cast<uint32_t>(me < d ? me : me - 1) * kSlotBytes + row_off,
                                                  static_cast<uint32_t>(d));
          const uint32_t remote_bar = ptx::map_to_cta(red_full_u32, static_cast<uint32_t>(d));
          if (row_ok) {
#pragma unroll
            for (int c4 = 0; c4 < HW / 4; ++c4) {
              const uint32_t c = static_cast<uint32_t>((half * HW) / 4 + c4);
              if (empty_split)
                ptx::st_async_v4(remote + ((c ^ swz) << 4), 0u, 0u, 0u, 0u, remote_bar);
              else
                ptx::st_async_v4(remote + ((c ^ swz) << 4), snd[dd - 1][4 * c4], snd[dd - 1][4 * c4 + 1],
                                 snd[dd - 1][4 * c4 + 2], snd[dd - 1][4 * c4 + 3], remote_bar);
            }
          }
        }
        float own[HW];
        {
          uint32_t v[HW];
#pragma unroll
          for (int c8 = 0; c8 < HW / 8; ++c8) ptx::tmem_ld_32x32b_x8(acc_addr + me * W + c8 * 8, &v[c8 * 8]);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < HW; ++i) own[i] = empty_split ? 0.0f : __uint_as_float(v[i]);
        }
        release_accumulator();
        if (!ptx::mbar_wait_cluster(red_full_u32, static_cast<uint32_t>(tile_iter) & 1u, abort_flag, kWaitPartials,
                                    wait_limit))
          break;
        float sum[HW];
#pragma unroll
        for (int s = 0; s < S; ++s) {
          if (s == me) {
#pragma unroll
            for (int i = 0; i < HW; ++i) sum[i] = s == 0 ? own[i] : __fadd_rn(sum[i], own[i]);
          } else {
            const uint32_t slot = red_u32 + static_cast<uint32_t>(s < me ? s : s - 1) * kSlotBytes + row_off;
#pragma unroll
            for (int c4 = 0; c4 < HW / 4; ++c4) {
              const uint32_t c = static_cast<uint32_t>((half * HW) / 4 + c4);
              const uint4 v = row_ok ? ptx::ld_shared_v4(slot + ((c ^ swz) << 4)) : make_uint4(0u, 0u, 0u, 0u);
              const float f[4] = {__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w)};
#pragma unroll
              for (int i = 0; i < 4; ++i) sum[c4 * 4 + i] = s == 0 ? f[i] : __fadd_rn(sum[c4 * 4 + i], f[i]);
            }
          }
        }
        {
          __half* dst = static_cast<__half*>(p.out) + out_row * p.out_ld + t.nt * BN + me * W + half * HW;
          const int cbase = t.nt * BN + me * W + half * HW;
#pragma unroll
          for (int i = 0; i < HW / 8; ++i) {
            if (row_ok && cbase + 8 * i < p.n) {
              uint4 o;
              o.x = pack_half2(sum[8 * i] * alpha, sum[8 * i + 1] * alpha);
              o.y = pack_half2(sum[8 * i + 2] * alpha, sum[8 * i + 3] * alpha);
              o.z = pack_half2(sum[8 * i + 4] * alpha, sum[8 * i + 5] * alpha);
              o.w = pack_half2(sum[8 * i + 6] * alpha, sum[8 * i + 7] * alpha);
              *reinterpret_cast<uint4*>(dst + 8 * i) = o;
            }
          }
        }
        if (task + num_workers < total_tasks) {     // another tile follows: hand the slots back
          ptx::fence_acq_rel_cluster();      // every lane's reads of the slots, before lane 0 reports them
          __syncwarp();
          if (lane == 0) {
#pragma unroll
            for (int dd = 1; dd < S; ++dd)
              ptx::mbar_arrive_release_cluster(ptx::map_to_cta(red_empty_u32, static_cast<uint32_t>((me + dd) % S)));
          }
        }
      } else if constexpr (kSwiGlu) {
        // Accumulator columns 0..127 are the gate, 128..255 the up projection of the same 128
        // intermediate columns. This warp takes 64 of them (4 blocks of 16). Both operands are
        // rounded to FP16 first - the values the unfused path would have written and read back - and
        // that is also how they wait in registers (64 packed words): the whole slab is read before
        // any arithmetic, the 64 columns shared with the other accumulator first, so the accumulator
        // goes back to the MMA warp at once and silu(gate) * up + the quantisation of one tile run
        // while the next tile is being computed.
        const uint32_t g_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                static_cast<uint32_t>(acc * Cfg::kAccStride + half * 64);
        uint32_t gp[32], up[32];    // gate / up columns 0..63 of this warp as half2 pairs
        auto load_half = [&](uint32_t addr, uint32_t* packed) {
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(addr, v);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i)
            packed[i] = pack_half2(__uint_as_float(v[2 * i]) * alpha, __uint_as_float(v[2 * i + 1]) * alpha);
        };
        if (reversed) {     // accumulator 0: the shared columns are up columns 64..127 of the tile (second half's)
          load_half(g_addr + 128, up);
          load_half(g_addr + 160, up + 16);
          release_overlap();
          load_half(g_addr, gp);
          load_half(g_addr + 32, gp + 16);
        } else {            // accumulator 1: gate columns 0..63 of the tile (first half's)
          load_half(g_addr, gp);
          load_half(g_addr + 32, gp + 16);
          release_overlap();
          load_half(g_addr + 128, up);
          load_half(g_addr + 160, up + 16);
        }
        release_accumulator();
        // Rows behind the end of the group hold whatever the neighbouring rows of A and the unwritten
        // part of the scale region made of them - possibly NaN or infinity, which send every division
        // below down its slow path. A slab without a valid row is skipped, and the lanes of invalid
        // rows compute on zeros.
        if (t.mt * kTileM + slab_row >= s_rows[t.g]) {
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1;
          continue;
        }
        if (!row_ok) {
#pragma unroll
          for (int i = 0; i < 32; ++i) { gp[i] = 0u; up[i] = 0u; }
        }
        uint32_t payload[8];
        uint32_t scale_word = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          float gv[16], uv[16], v[16];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const __half2 g2 = *reinterpret_cast<const __half2*>(&gp[8 * b + i]);
            const __half2 u2 = *reinterpret_cast<const __half2*>(&up[8 * b + i]);
            gv[2 * i] = __low2float(g2);
            gv[2 * i + 1] = __high2float(g2);
            uv[2 * i] = __low2float(u2);
            uv[2 * i + 1] = __high2float(u2);
          }
          silu_mul_block16(gv, uv, v);
          uint32_t lo, hi;
          const uint8_t code = quantize_block16(v, lo, hi);
          payload[2 * b] = lo;
          payload[2 * b + 1] = hi;
          scale_word |= static_cast<uint32_t>(code) << (8 * b);
        }
        if (row_ok) {
          const int inter = p.swiglu_inter;
          const int col = t.nt * 128 + half * 64;                 // first intermediate column of this lane's 64
          uint4* dst = reinterpret_cast<uint4*>(p.q_out + out_row * (inter >> 1) + (col >> 1));
          dst[0] = make_uint4(payload[0], payload[1], payload[2], payload[3]);
          dst[1] = make_uint4(payload[4], payload[5], payload[6], payload[7]);
          const int row_in_group = t.mt * kTileM + row_in_tile;
          *reinterpret_cast<uint32_t*>(p.q_scale + t.g * p.q_scale_group_stride +
                                       sf_offset(row_in_group, col >> 4, (inter + 63) >> 6)) = scale_word;
        }
      } else if constexpr (kOutF32) {
        float* dst = static_cast<float*>(p.out) + t.split * p.out_split_stride + out_row * p.out_ld + col0;
        constexpr int kF32Chunks = kWarpCols / 32;
#pragma unroll 1
        for (int ci = 0; ci < kF32Chunks; ++ci) {
          const int c = reversed ? kF32Chunks - 1 - ci : ci;
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(taddr + c * 32, v);
          ptx::tmem_ld_wait();
          if (kOverlap && ci == 1) release_overlap();     // two chunks = the 64 shared columns
          if (ci == kF32Chunks - 1) release_accumulator();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = empty_split ? 0u : __float_as_uint(__uint_as_float(v[i]) * alpha);
          if (staged) {
            if (col0 + c * 32 < p.n) {
              wait_staging_free();
              fill_staging(v);
              store_staging(col0 + c * 32);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (row_ok && col0 + c * 32 + 4 * i < p.n)
                *reinterpret_cast<uint4*>(dst + c * 32 + 4 * i) = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            }
          }
        }
      } else {
        __half* dst = static_cast<__half*>(p.out) + out_row * p.out_ld + col0;
        constexpr int kChunkCols = kWarpCols >= 64 ? 64 : kWarpCols;     // columns per pass
        constexpr int kChunks = kWarpCols / kChunkCols;
        const bool plain = !empty_split && alpha == 1.0f;   // warp-uniform: no scaling needed
        // 32 accumulator columns -> 16 packed half2 words
        auto load_pack = [&](int col, uint32_t* packed) {
          uint32_t v[kLdCols];
          ptx::tmem_ld_32x32b_x32(taddr + col, v);
          ptx::tmem_ld_wait();
          if (plain) {
#pragma unroll
            for (int i = 0; i < kLdCols / 2; ++i)
              packed[i] = pack_half2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
          } else {
#pragma unroll
            for (int i = 0; i < kLdCols / 2; ++i)
              packed[i] = empty_split ? 0u
                                      : pack_half2(__uint_as_float(v[2 * i]) * alpha,
                                                   __uint_as_float(v[2 * i + 1]) * alpha);
          }
        };
        auto direct_store = [&](int c, const uint32_t* packed) {
#pragma unroll
          for (int i = 0; i < kChunkCols / 8; ++i) {
            if (row_ok && col0 + c * kChunkCols + 8 * i < p.n)
              *reinterpret_cast<uint4*>(dst + c * kChunkCols + 8 * i) =
                  make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
          }
        };
        const bool use_staging = kChunkCols == 64 && staged;
        if constexpr (kChunks == 2 && kChunkCols == 64) {
          // 128 columns per warp: the whole slab is converted into registers first, so the
          // accumulator goes back to the MMA warp before any output leaves the registers; the 64
          // columns shared with the other accumulator are read first and handed back at once
          uint32_t p0[32], p1[32];
          if (reversed) {
            load_pack(96, p1 + 16);
            load_pack(64, p1);
            release_overlap();
            load_pack(32, p0 + 16);
            load_pack(0, p0);
          } else {
            load_pack(0, p0);
            load_pack(32, p0 + 16);
            release_overlap();
            load_pack(64, p1);
            load_pack(96, p1 + 16);
          }
          release_accumulator();
          if (use_staging) {
            wait_staging_free();
            if (col0 < p.n) { fill_staging(p0); store_staging(col0); }
            if (col0 + 64 < p.n) {
              wait_staging_free();
              fill_staging(p1);
              store_staging(col0 + 64);
            }
          } else {
            direct_store(0, p0);
            direct_store(1, p1);
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < kChunks; ++c) {
            uint32_t packed[32];
#pragma unroll
            for (int h = 0; h < kChunkCols / kLdCols; ++h) load_pack(c * kChunkCols + h * kLdCols, packed + 16 * h);
            if (c == kChunks - 1) release_accumulator();
            const int col = col0 + c * kChunkCols;
            if (use_staging) {
              if (col < p.n) {
                wait_staging_free();
                fill_staging(packed);
                store_staging(col);
              }
            } else {
              direct_store(c, packed);
            }
          }
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    // shared memory must outlive the last box
    if (lane == 0) ptx::bulk_wait_group<0>();
    __syncwarp();
  }

  // ---- teardown
  if constexpr (kSplitCluster) {
    if (warp < kFirstEpilogueWarp) ptx::cluster_wait();   // the epilogue warps did so before their first tile
  }
  __syncthreads();
  // In a pair neither CTA may leave (or free tensor memory) while the other can still
  // signal its barriers or read its shared memory.
  if constexpr (kTwoCta || kSplitCluster) ptx::cluster_sync();
  const int aborted = *abort_flag;
  if (aborted != 0) {
    // give copies that may still be in flight time to land before shared memory goes away
    long long start = clock64();
    while (clock64() - start < (1ll << 22)) {
    }
    if (threadIdx.x == 0 && p.error) atomicCAS(p.error, 0, aborted | (static_cast<int>(blockIdx.x) << 8));
  }
  if (warp == kWarpMma) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc<kCtas>(tmem_base, Cfg::kTmemCols);
  }
}

}  // namespace b200
