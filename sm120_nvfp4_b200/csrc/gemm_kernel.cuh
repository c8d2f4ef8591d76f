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
//                      CTAs and fits a deeper pipeline. No multicast load is used anywhere.
//
// Structure of one CTA (640 threads, one CTA per SM):
//   warps 0, 2  loaders: TMA loads of the A tile / the B tile (128-byte swizzle) into a ring
//               of shared-memory stages
//   warp 3      scale loader: untiled bulk copies of the stage's scale atoms
//   warps 4-11  scale movers, two teams of one warp per TMEM lane quarter: read the landed atoms
//               from shared memory and write them into the k-stage's tensor-memory buffer with
//               tcgen05.st (two wide stores per stage instead of a dozen tcgen05.cp), ahead of
//               the MMAs. One k-stage costs a mover ~700 cycles of waits, loads, stores and
//               arrives against ~520 cycles of MMA work, so the teams take alternate k-stages.
//   warp 1      MMA issuer (first CTA of a pair only): tcgen05.mma kind::mxf4nvf4
//               (M x BN x 64 per instruction) accumulates FP32 in tensor memory;
//               tcgen05.commit releases the stage / publishes the tile
//   warps 12-19 epilogue: tcgen05.ld of the accumulator (a 32-lane quarter and half of the
//               columns per warp), conversion, 16-byte stores with row / column predicates
// All mbarrier waits are bounded (ptx::mbar_wait); a timeout is reported through
// GemmParams::error instead of hanging.
#pragma once

#include <cuda_fp16.h>

#include "nvfp4_math.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr int kBlockM = 128;        // rows of A per CTA = rows of one UMMA half
constexpr int kStageKBytes = 128;   // bytes of K per stage row = one swizzle span
constexpr int kStageK = 256;        // E2M1 values of K per stage
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
constexpr int kFirstSfMoverWarp = 4;    // two teams of four warps (one warp per TMEM lane quarter)
constexpr int kSfMoverTeams = 2;        // team t moves the scales of k-stages t, t + 2, t + 4, ...
constexpr int kFirstEpilogueWarp = kFirstSfMoverWarp + 4 * kSfMoverTeams;
constexpr int kGemmThreads = 32 * (kFirstEpilogueWarp + kEpilogueWarps);
constexpr int kMaxStages = 8;
constexpr int kMaxSfSlots = 16;
constexpr int kBarrierBytes = 512;      // 2 x kMaxStages + 2 x kMaxSfSlots + 4 mbarriers, TMEM base, abort flag
constexpr int kSmemBudget = 232448;     // 227 KB opt-in limit per CTA

struct GemmParams {
  int num_groups;
  int n;                      // output columns per group
  int k;                      // logical K
  int m_uniform;              // rows per group when seqlens == nullptr
  const int* seqlens;         // [G] valid rows per group (device) or nullptr
  const int* cu_seqlens;      // [G+1] first row of each group (device) or nullptr
  const uint8_t* sfa;
  const uint8_t* sfb;
  int sfa_atom_rows;          // 128-row atom rows in one group's SFA region
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
  int a_sub_bytes;            // shared-memory bytes of one sub-stage of A: rows in the A box x 128
  int num_stages;             // depth of the operand ring in shared memory (<= kMaxStages)
  int num_sf_slots;           // depth of the scale-atom ring in shared memory (<= kMaxSfSlots)
  int tma_store;              // 1: the output tensor map is valid, full 32-row slabs go out by TMA store
  int out_rows_per_split;     // rows between split-K slices in the output tensor map (M), 0 without split
  // Fused gate/up variant (kSwiGlu kernels): B holds [gate rows 0..I) ; up rows I..2I) per group, a
  // tile computes 128 gate and the matching 128 up columns, and the epilogue writes
  // NVFP4(silu(gate) * up) instead of the FP16 product.
  int swiglu_inter;           // I (multiple of 128), 0 for plain GEMMs
  uint8_t* q_out;             // packed E2M1 [rows, I/2]
  uint8_t* q_scale;           // UE4M3 scale regions, one per group, indexed by the row inside the group
  long long q_scale_group_stride;
  // Debug switches (environment variable B200_NVFP4_DEBUG, 0 in production). Bits 1, 2, 4 and 8
  // switch parts of the kernel off to find what bounds it - results are then wrong by design:
  // 1 no MMAs (data path only), 2 no operand loads (barriers only), 4 no tensor-memory stores of
  // the scales, 8 no scale loads. Bit 64 records time stamps into `trace`.
  int debug;
  unsigned long long* trace;  // optional time-stamp buffer (debug bit 64), else nullptr
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
  static constexpr int kAccStages = BN <= 128 ? 2 : 1;
  // Tensor memory: accumulator stage(s) first, then a ring of scale-factor buffers, one per
  // k-stage in flight, so the scale copies of a k-stage can be issued (by their own warps)
  // while the MMAs of earlier stages are still running. The ring is as deep as the columns
  // allow, but never deeper than the operand ring (kernel: sf_depth).
  // Sub-stages per pipeline stage. One sub-stage is 256 k-values (one 128-byte swizzle span, four
  // MMAs). A barrier round - waits, arrivals, commit, the scale movers' pass - costs several
  // hundred cycles whatever it carries, and an MMA costs its issuing thread ~50 cycles however
  // narrow it is; for 64-column tiles (skinny problems, bound by streaming B) two sub-stages per
  // round halve the rounds per byte.
  static constexpr int kSub = BN == 64 ? 2 : 1;
  static constexpr int kAtomsPerStage = 4 * kSub;
  static constexpr int kSfColsPerSub = 16 + 4 * kSfbColsPerMma;   // 4 MMAs: SFA 4x4, SFB 4xN/32
  static constexpr int kSfColsPerBuf = kSub * kSfColsPerSub;
  static constexpr int kSfBase = kAccStages * BN;
  static constexpr int kMaxSfBufs = (512 - kSfBase) / kSfColsPerBuf;
  static constexpr int kTmemCols = 512;
  // One sub-stage of A: 128 rows, or fewer when the whole problem has fewer rows (the loader's box
  // then covers round-up-to-8 rows; the MMA still reads 128 rows' worth of shared memory, the rest
  // being whatever follows - rows that are never stored). The freed space deepens the ring, which
  // is what a skinny problem needs: it is bound by the bytes of B in flight.
  static constexpr int kABytes = kBlockM * kStageKBytes;
  static constexpr int kBBytes = kBRows * kStageKBytes;            // one sub-stage of B
  static constexpr int kSfaBytes = 4 * kAtomBytes;                 // one sub-stage of SFA atoms
  static constexpr int kSfbBytes = kSfbGroups * 4 * kAtomBytes;
  // stage layout: [A sub-stages][B sub-stages]; slot layout: [SFA atoms][SFB atoms of group 0][group 1]
  __host__ __device__ static constexpr int stage_bytes(int a_sub_bytes) { return kSub * (a_sub_bytes + kBBytes); }
  static constexpr int kSfSlotBytes = kSub * (kSfaBytes + kSfbBytes);  // one slot of the scale-atom ring
  // Output staging for TMA stores: 32 rows x 128 bytes per epilogue warp. Tiles of 64 columns
  // give a warp only 32 columns (64 bytes of FP16 per row) and keep the direct-store epilogue.
  static constexpr int kStagingWarpBytes = 32 * 128;
  static constexpr int kStagingBytes = BN >= 128 ? kEpilogueWarps * kStagingWarpBytes : 0;

  // Shared memory: [operand stages][output staging][scale slots][barriers][group tables]; +1024 slack to align
  // the base. The scale atoms have a ring of their own: a slot is free again as soon as the
  // movers have read it into registers, so scale loads (small, long-latency bulk copies) run
  // well ahead of the operand ring instead of waiting for MMAs to release a stage.
  static constexpr int fixed_bytes(int num_groups) {
    return 1024 + kBarrierBytes + 3 * (num_groups + 1) * 4 + kStagingBytes;
  }
  static constexpr int kMinSfSlots = 4;
  static constexpr int stages_for(int num_groups, int a_sub_bytes = kABytes) {
    // as many operand stages as fit beside a minimum of scale slots; the MMA reads a full 128-row
    // A block from the last sub-stage, so that much shared memory must follow it
    int s = (kSmemBudget - fixed_bytes(num_groups) - kMinSfSlots * kSfSlotBytes) / stage_bytes(a_sub_bytes);
    return s > kMaxStages ? kMaxStages : s;
  }
  static constexpr int sf_slots_for(int num_groups, int a_sub_bytes = kABytes) {
    int n = (kSmemBudget - fixed_bytes(num_groups) - stages_for(num_groups, a_sub_bytes) * stage_bytes(a_sub_bytes)) /
            kSfSlotBytes;
    return n > kMaxSfSlots ? kMaxSfSlots : n;
  }
  static constexpr int smem_bytes(int num_groups, int a_sub_bytes = kABytes) {
    return fixed_bytes(num_groups) + stages_for(num_groups, a_sub_bytes) * stage_bytes(a_sub_bytes) +
           sf_slots_for(num_groups, a_sub_bytes) * kSfSlotBytes;
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

// Debug time stamps: trace[((cta * 8 + role) * 64 + iter) * 2 + which] = SM clock counter.
__device__ __forceinline__ void trace_stamp(const GemmParams& p, int role, int iter, int which) {
  if ((p.debug & 64) && p.trace != nullptr && blockIdx.x < 2 && iter < 64) {
    const unsigned long long t = static_cast<unsigned long long>(clock64());
    p.trace[((blockIdx.x * 8 + role) * 64 + iter) * 2 + which] = t;
  }
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int BN, bool kOutF32, bool kTwoCta, bool kSwiGlu = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                  const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_out, const GemmParams p) {
  using Cfg = GemmCfg<BN, kTwoCta>;
  static_assert(!kSwiGlu || (BN == 256 && !kOutF32), "the fused gate/up epilogue is built on 256-column FP16 tiles");
  if ((p.debug & 64) && p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long ns;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
    p.trace[((0 * 8 + 7) * 64 + 61) * 2 + 0] = static_cast<unsigned long long>(clock64());
    p.trace[((0 * 8 + 7) * 64 + 61) * 2 + 1] = ns;
  }
  constexpr int kCtas = Cfg::kCtas;
  constexpr int kAccStages = Cfg::kAccStages;
  constexpr int kTileM = Cfg::kTileM;
  const int kStages = p.num_stages;
  // k-stages whose scales may sit in tensor memory at once. Not more than operand stages: a
  // mover that ran further ahead would arrive on a stage's `full` barrier before the stage's
  // previous use had completed.
  const int sf_depth = Cfg::kMaxSfBufs < kStages ? Cfg::kMaxSfBufs : kStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* stage_base = smem;
  const int kSfSlots = p.num_sf_slots;
  const uint32_t a_bytes = static_cast<uint32_t>(p.a_sub_bytes);
  const uint32_t stage_bytes = static_cast<uint32_t>(Cfg::stage_bytes(p.a_sub_bytes));
  uint8_t* staging_base = smem + kStages * stage_bytes;   // 1024-byte aligned: stages are multiples of 1 KB
  uint8_t* sf_base = staging_base + Cfg::kStagingBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sf_base + kSfSlots * Cfg::kSfSlotBytes);
  // full:      the stage is ready for the MMAs: its A / B tiles landed in shared memory and
  //            its scales are in tensor memory (pair: in both CTAs; lives in the first CTA).
  //            One barrier, because every wait costs the MMA issuer ~150 cycles of a
  //            ~520-cycle stage.
  // empty:     the MMAs that read the stage are done
  // sf_landed: a slot of the scale ring received its atoms
  // sf_free:   the moving team has read the slot into registers and the other team has seen it land
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* sf_landed_bar = empty_bar + kMaxStages;
  uint64_t* sf_free_bar = sf_landed_bar + kMaxSfSlots;
  uint64_t* acc_full_bar = sf_free_bar + kMaxSfSlots;
  uint64_t* acc_empty_bar = acc_full_bar + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty_bar + 2);
  int* abort_flag = reinterpret_cast<int*>(tmem_holder + 1);
  int* s_cu_tiles = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(full_bar) + kBarrierBytes);
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
  const int worker = static_cast<int>(blockIdx.x) / kCtas;     // CTA or CTA pair
  const int num_workers = static_cast<int>(gridDim.x) / kCtas;

  // ---- group tables: valid rows, first row and m-tile prefix of every group
  for (int g = threadIdx.x; g < G; g += kGemmThreads) {
    int rows = p.seqlens ? p.seqlens[g] : p.m_uniform;
    rows = rows > 0 ? rows : 0;
    s_rows[g] = rows;
    s_row0[g] = p.cu_seqlens ? p.cu_seqlens[g] : g * p.m_uniform;
    s_cu_tiles[g] = (rows + kTileM - 1) / kTileM;
  }
  // Set-up runs in parallel: the lanes of warp 0 initialise one barrier each, the MMA warp
  // allocates tensor memory meanwhile. A single problem (one group) needs no scan of tile counts
  // and therefore only one block-wide barrier before the pipeline starts.
  if (warp == 0) {
    if (lane == 0) *abort_flag = 0;
    for (int s = lane; s < kStages; s += 32) {
      // arrivals: the A and the B loader of the owning CTA + every scale-mover warp of a team
      ptx::mbar_init(full_bar + s, 2 + 4 * kCtas);
      ptx::mbar_init(empty_bar + s, 1);
    }
    for (int s = lane; s < kSfSlots; s += 32) {
      ptx::mbar_init(sf_landed_bar + s, 1);
      ptx::mbar_init(sf_free_bar + s, 4 * kSfMoverTeams);   // every mover warp, see the movers
    }
    if (lane < 2) {
      ptx::mbar_init(acc_full_bar + lane, 1);
      ptx::mbar_init(acc_empty_bar + lane, kEpilogueWarps * kCtas);
    }
    __syncwarp();
    if (lane == 0) {
      ptx::fence_barrier_init();
      ptx::prefetch_tensormap(&tmap_a);
      ptx::prefetch_tensormap(&tmap_b);
      if (p.tma_store) ptx::prefetch_tensormap(&tmap_out);
    }
  } else if (warp == kWarpMma) {
    ptx::tmem_alloc<kCtas>(tmem_holder, Cfg::kTmemCols);
    ptx::tmem_relinquish<kCtas>();
  }
  if (G == 1) {
    if (threadIdx.x == 0) {   // this thread wrote the only table entry itself
      const int tiles = s_cu_tiles[0];
      s_cu_tiles[0] = 0;
      s_cu_tiles[1] = tiles;
      if (blockIdx.x == 0) {
        const int t128 = (s_rows[0] + kBlockM - 1) / kBlockM;
        if (p.tiles_out) p.tiles_out[0] = t128;
        if (p.cu_tiles_out) { p.cu_tiles_out[0] = 0; p.cu_tiles_out[1] = t128; }
      }
    }
  } else {
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
  ptx::tc_fence_before_sync();
  __syncthreads();
  if constexpr (kTwoCta) ptx::cluster_sync();  // the partner's barriers are initialised too
  ptx::tc_fence_after_sync();

  if ((p.debug & 64) && p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long ns;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
    p.trace[((0 * 8 + 7) * 64 + 63) * 2 + 0] = static_cast<unsigned long long>(clock64());
    p.trace[((0 * 8 + 7) * 64 + 63) * 2 + 1] = ns;
  }
  const uint32_t tmem_base = *tmem_holder;
  const int total_mt = s_cu_tiles[G];
  // fused gate/up: a tile covers 128 columns of the intermediate (its gate and its up half)
  const int n_tiles = kSwiGlu ? p.swiglu_inter / 128 : (p.n + BN - 1) / BN;
  const int total_tasks = total_mt * n_tiles * p.num_splits;
  const int kt = (p.k + 63) / 64;               // scale atoms along K
  constexpr int kSub = Cfg::kSub;
  constexpr int kAtomsPerStage = Cfg::kAtomsPerStage;
  const int k_stages = (kt + kAtomsPerStage - 1) / kAtomsPerStage;   // pipeline stages along K
  const int n_sf_tiles = (p.n + 127) / 128;     // 128-row scale tiles of B

  // 32-bit shared-window addresses of the rings: the role loops below advance them with adds.
  const uint32_t stage_u32 = ptx::smem_u32(stage_base);
  const uint32_t sf_u32 = ptx::smem_u32(sf_base);
  const uint32_t full_u32 = ptx::smem_u32(full_bar);
  const uint32_t empty_u32 = ptx::smem_u32(empty_bar);
  const uint32_t sf_landed_u32 = ptx::smem_u32(sf_landed_bar);
  const uint32_t sf_free_u32 = ptx::smem_u32(sf_free_bar);
  // where arrivals for a stage's `full` barrier go: this CTA's barrier, or the leader's
  const uint32_t full_target_u32 = kTwoCta ? ptx::map_to_cta(full_u32, 0) : full_u32;
  const bool tracing = (p.debug & 64) != 0 && p.trace != nullptr && blockIdx.x < 2;
  const int k_stages_full = kt / kAtomsPerStage;   // k-stages with all their atoms

  if (warp == kWarpLoadA || warp == kWarpLoadB) {
    // ============================ operand loaders ============================
    // One thread per operand. Completion bytes are counted on the barrier of the first CTA
    // (in a pair both CTAs' loads report there, and only the first CTA's loader arms it, for
    // both halves), so the MMA issuer waits on one barrier per stage.
    {
      const bool is_a = warp == kWarpLoadA;
      const CUtensorMap* tmap = is_a ? &tmap_a : &tmap_b;
      const uint32_t bytes = is_a ? a_bytes : Cfg::kBBytes;
      const uint32_t dst0 = stage_u32 + (is_a ? 0 : kSub * a_bytes);
      const bool no_loads = (p.debug & 2) != 0;   // experiment: barriers only
      int stage = 0, iter = 0;
      uint32_t phase = 0, dst = dst0, full_a = full_u32, full_t = full_target_u32, empty_a = empty_u32;
      bool ok = true;
      for (int task = worker; task < total_tasks && ok; task += num_workers) {
        TileCoord t = decode_tile(task, total_mt, n_tiles, p.num_splits, p.raster_m, s_cu_tiles, G);
        int row;
        if (is_a) row = s_row0[t.g] + t.mt * kTileM + static_cast<int>(cta_rank) * kBlockM;
        else if constexpr (kSwiGlu) row = t.g * p.b_group_rows + t.nt * 128 + (kTwoCta ? static_cast<int>(cta_rank) * p.swiglu_inter : 0);
        else row = t.g * p.b_group_rows + t.nt * BN + static_cast<int>(cta_rank) * Cfg::kBRows;
        const int ks_begin = (k_stages * t.split) / p.num_splits;
        const int ks_end = (k_stages * (t.split + 1)) / p.num_splits;
        int c0 = ks_begin * kSub * kStageKBytes;
        for (int ks = ks_begin; ks < ks_end; ++ks, c0 += kSub * kStageKBytes) {
          if (tracing && lane == 0) trace_stamp(p, is_a ? 0 : 4, iter, 0);
          if (!ptx::mbar_wait(empty_a, phase ^ 1, abort_flag, 1)) { ok = false; break; }
          if (tracing && lane == 0) trace_stamp(p, is_a ? 0 : 4, iter, 1);
          ++iter;
          if (ptx::elect_one()) {
            if (no_loads) {
              if (leader) ptx::mbar_arrive(full_a);
            } else if constexpr (kTwoCta) {
              if (leader) ptx::mbar_arrive_expect_tx(full_a, 2 * kSub * bytes);
#pragma unroll
              for (int sub = 0; sub < kSub; ++sub)
                ptx::tma_load_2d_pair(dst + sub * bytes, tmap, full_t, c0 + sub * kStageKBytes, row);
            } else {
              // a sub-stage that starts behind the end of K is filled with zeros by the load
              ptx::mbar_arrive_expect_tx(full_a, kSub * bytes);
              if (kSwiGlu && !is_a) {   // 128 gate rows, then the 128 up rows I further down (128-row box)
                ptx::tma_load_2d(dst, tmap, full_a, c0, row);
                ptx::tma_load_2d(dst + bytes / 2, tmap, full_a, c0, row + p.swiglu_inter);
              } else {
#pragma unroll
                for (int sub = 0; sub < kSub; ++sub)
                  ptx::tma_load_2d(dst + sub * bytes, tmap, full_a, c0 + sub * kStageKBytes, row);
              }
            }
          }
          dst += stage_bytes; full_a += 8; full_t += 8; empty_a += 8;
          if (++stage == kStages) {
            stage = 0; phase ^= 1; dst = dst0; full_a = full_u32; full_t = full_target_u32; empty_a = empty_u32;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == kWarpLoadSf) {
    // ============================== scale loader =============================
    // Fills the scale-atom ring: waits for a slot the movers have drained, then bulk-copies
    // the k-stage's SFA atoms and SFB atoms into it.
    {
      const bool no_loads = (p.debug & 8) != 0;   // experiment: no scale traffic
      int slot = 0, iter = 0;
      uint32_t phase = 0, dst = sf_u32, landed_a = sf_landed_u32, free_a = sf_free_u32;
      bool ok = true;
      for (int task = worker; task < total_tasks && ok; task += num_workers) {
        TileCoord t = decode_tile(task, total_mt, n_tiles, p.num_splits, p.raster_m, s_cu_tiles, G);
        const int sf_tile0 = kSwiGlu ? t.nt : (t.nt * BN) / 128;
        int sfb_groups = Cfg::kSfbGroups;
        if (!kSwiGlu && sf_tile0 + sfb_groups > n_sf_tiles) sfb_groups = n_sf_tiles - sf_tile0;
        const int ks_begin = (k_stages * t.split) / p.num_splits;
        const int ks_end = (k_stages * (t.split + 1)) / p.num_splits;
        // A slab that lies wholly behind the group's scale region (second CTA of a pair on a short
        // group or matrix) has no scales of its own; its rows are never stored, so it reads the
        // region's last atom row instead of memory past the region.
        int sfa_row = t.mt * kCtas + static_cast<int>(cta_rank);
        if (sfa_row >= p.sfa_atom_rows) sfa_row = p.sfa_atom_rows - 1;
        const uint8_t* sfa_src = p.sfa + t.g * p.sfa_group_stride +
                                 (static_cast<long long>(sfa_row) * kt + ks_begin * kAtomsPerStage) * kAtomBytes;
        const uint8_t* sfb_src = p.sfb + t.g * p.sfb_group_stride +
                                 (static_cast<long long>(sf_tile0) * kt + ks_begin * kAtomsPerStage) * kAtomBytes;
        // second 128-row scale tile of the B tile: the next one, or the up half's (I / 128 tiles on)
        const long long sfb_group_step = static_cast<long long>(kSwiGlu ? p.swiglu_inter / 128 : 1) * kt * kAtomBytes;
        for (int ks = ks_begin; ks < ks_end;
             ++ks, sfa_src += kAtomsPerStage * kAtomBytes, sfb_src += kAtomsPerStage * kAtomBytes) {
          if (!ptx::mbar_wait(free_a, phase ^ 1, abort_flag, 8)) { ok = false; break; }
          if (tracing && lane == 0) trace_stamp(p, 2, iter, 0);
          const uint32_t sf_bytes = ks < k_stages_full ? static_cast<uint32_t>(kAtomsPerStage) * kAtomBytes
                                                       : static_cast<uint32_t>(kt - ks * kAtomsPerStage) * kAtomBytes;
          if (ptx::elect_one()) {
            if (no_loads) {
              ptx::mbar_arrive(landed_a);
            } else {
              ptx::mbar_arrive_expect_tx(landed_a, sf_bytes * (1 + sfb_groups));
              ptx::bulk_load(dst, sfa_src, sf_bytes, landed_a);
              ptx::bulk_load(dst + kSub * Cfg::kSfaBytes, sfb_src, sf_bytes, landed_a);
              if (Cfg::kSfbGroups == 2 && sfb_groups == 2)
                ptx::bulk_load(dst + kSub * Cfg::kSfaBytes + kAtomsPerStage * kAtomBytes, sfb_src + sfb_group_step,
                               sf_bytes, landed_a);
            }
          }
          if (tracing && lane == 0) trace_stamp(p, 2, iter, 1);
          ++iter;
          dst += Cfg::kSfSlotBytes; landed_a += 8; free_a += 8;
          if (++slot == kSfSlots) { slot = 0; phase ^= 1; dst = sf_u32; landed_a = sf_landed_u32; free_a = sf_free_u32; }
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
      const uint32_t sf_col0 = tmem_base + Cfg::kSfBase;
      const bool no_mma = (p.debug & 1) != 0;   // experiment: data path only
      int stage = 0, acc = 0, iter = 0, sfbuf = 0;
      uint32_t phase = 0, acc_phase = 0, full_a = full_u32, empty_a = empty_u32, a_lo = a_lo0, sf_col = sf_col0;
      bool ok = true;
      for (int task = worker; task < total_tasks && ok; task += num_workers) {
        TileCoord t = decode_tile(task, total_mt, n_tiles, p.num_splits, p.raster_m, s_cu_tiles, G);
        const int ks_begin = (k_stages * t.split) / p.num_splits;
        const int ks_end = (k_stages * (t.split + 1)) / p.num_splits;
        // A tile narrower than 128 columns uses part of a 128-row scale atom: column
        // (n0 % 128) / 32 of the four TMEM columns the atom occupies.
        const uint32_t sfb_sub = BN < 128 ? static_cast<uint32_t>(((t.nt * BN) % 128) / 32) : 0u;
        if (tracing && lane == 0) trace_stamp(p, 7, iter / 32, 0);
        if (!ptx::mbar_wait(acc_empty_bar + acc, acc_phase ^ 1, abort_flag, 2)) break;
        if (tracing && lane == 0) trace_stamp(p, 7, iter / 32, 1);
        ptx::tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(acc * BN);
        // The tensor pipe accepts an MMA only when the previous one is almost done (issuing
        // four 128-cycle MMAs occupies this thread for 512 cycles), so whatever this thread does
        // between the last MMA of a k-stage and the first of the next must fit into one MMA's
        // run time or the pipe idles. The next stage's barrier is therefore probed between the
        // third and the fourth MMA, while the pipe is busy.
        bool ready = false;
        for (int ks = ks_begin; ks < ks_end; ++ks) {
          if (tracing && lane == 0) trace_stamp(p, 1, iter, 0);
          if (!ready && !ptx::mbar_wait(full_a, phase, abort_flag, 3)) { ok = false; break; }
          if (tracing && lane == 0) trace_stamp(p, 1, iter, 1);
          ptx::tc_fence_after_sync();
          const uint32_t b_lo = a_lo + kSub * a_desc_sub;
          const uint32_t sfb_col = sf_col + 16 + sfb_sub;
          const bool full_stage = ks < k_stages_full;
          const bool last_ring = stage + 1 == kStages;
          const uint32_t next_full = last_ring ? full_u32 : full_a + 8;
          const uint32_t next_phase = last_ring ? phase ^ 1 : phase;
          // MMA number i of the stage (sub-stage i / 4, atom i % 4): 64 E2M1 values = 32 bytes along K
          // are +2 in the descriptor's 16-byte address field; a sub-stage is one operand block further
          auto issue = [&](int i, uint32_t accumulate) {
            const int sub = i >> 2, j = i & 3;
            ptx::tc_mma_nvfp4<kCtas>(tmem_acc, a_lo + sub * a_desc_sub + 2 * j,
                                     b_lo + sub * (Cfg::kBBytes >> 4) + 2 * j, ptx::kKmajorSw128DescHi, idesc,
                                     sf_col + sub * Cfg::kSfColsPerSub + 4 * j,
                                     sfb_col + sub * Cfg::kSfColsPerSub + j * Cfg::kSfbColsPerMma, accumulate);
          };
          if (full_stage && !no_mma) {
            if (ptx::elect_one()) {
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
              const int atoms = no_mma ? 0 : kt - ks * kAtomsPerStage;
              for (int i = 0; i < atoms && i < kAtomsPerStage; ++i) issue(i, (i > 0 || ks > ks_begin) ? 1u : 0u);
              ptx::tc_commit<kCtas>(empty_a, kAllCtas);
            }
          }
          ++iter;
          sf_col += Cfg::kSfColsPerBuf;
          if (++sfbuf == sf_depth) { sfbuf = 0; sf_col = sf_col0; }
          full_a += 8; empty_a += 8; a_lo += kDescStep;
          if (++stage == kStages) { stage = 0; phase ^= 1; full_a = full_u32; empty_a = empty_u32; a_lo = a_lo0; }
        }
        if (!ok) break;
        if (ptx::elect_one()) ptx::tc_commit<kCtas>(acc_full_bar + acc, kAllCtas);
        if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp >= kFirstSfMoverWarp && warp < kFirstEpilogueWarp) {
    // ============================== scale movers =============================
    // Warp q of a team moves a k-stage's scale atoms from the scale ring in shared memory into
    // lanes 32q..32q+31 of the k-stage's tensor-memory buffer (the MMA wants every 32-lane
    // quarter to hold the same 16 bytes per lane: row r of an atom lives in lane r % 32,
    // column r / 32). Lane t reads the 16 bytes at offset 16 t of each atom.
    const int q = warp & 3;
    const int team = (warp - kFirstSfMoverWarp) >> 2;
    const bool no_store = (p.debug & 4) != 0;   // experiment: skip the tensor-memory stores
    const uint32_t lane_off = static_cast<uint32_t>(lane) * 16;
    const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(Cfg::kSfBase);
    int stage = 0, slot = 0, iter = 0, sfbuf = 0;
    int lag_stage = 0, ahead = 0;   // operand stage of the k-stage sf_depth back; k-stages walked so far (saturates)
    uint32_t lag_phase = 0, slot_phase = 0;
    uint32_t src = sf_u32 + lane_off, landed_a = sf_landed_u32, free_a = sf_free_u32, full_t = full_target_u32;
    uint32_t lag_a = empty_u32, taddr = taddr0;
    bool ok = true;
    for (int task = worker; task < total_tasks && ok; task += num_workers) {
      TileCoord t = decode_tile(task, total_mt, n_tiles, p.num_splits, p.raster_m, s_cu_tiles, G);
      const int ks_begin = (k_stages * t.split) / p.num_splits;
      const int ks_end = (k_stages * (t.split + 1)) / p.num_splits;
      for (int ks = ks_begin; ks < ks_end; ++ks) {
        // every warp walks all k-stages (ring positions and phases advance for both teams) but
        // works only on its team's
        const bool mine = (iter & (kSfMoverTeams - 1)) == team;
        const bool need_lag = ahead >= sf_depth;
        if (!need_lag) ++ahead;
        // Both teams wait for every k-stage's atoms, also the ones the other team moves: a
        // parity wait is only meaningful for a waiter that has seen the previous phase of the
        // same barrier complete. A team that looked at a slot's barrier only on its own turns
        // would, with an odd number of slots, skip every other phase, and when it ran ahead of
        // the other team it would take the older completed phase for the one it waits for (stale
        // scales, and a fifth arrival on a four-arrival `sf_free` phase).
        if (!ptx::mbar_wait(landed_a, slot_phase, abort_flag, 5)) { ok = false; break; }
        // The reverse hazard: a warp that falls behind must still find the phase it waits for. If only
        // the moving team released the slot, the loader could refill it (phase n + 1, a k-stage the
        // lagging team has to move) before a lagging warp had looked at phase n; that warp would then
        // wait for phase n + 2, which needs its own release first - a deadlock. So the slot is handed
        // back by all mover warps: the other team's release says "seen", not "read".
        if (!mine && ptx::elect_one()) ptx::mbar_arrive(free_a);
        if (mine) {
          // 1. atoms of this k-stage: shared memory -> registers. Every lane polls: a
          //    single-lane wait costs a vote and a broadcast per call.
          if (tracing && q == 0 && lane == 0) trace_stamp(p, 3, iter, 0);
          const int atoms = ks < k_stages_full ? kAtomsPerStage : kt - ks * kAtomsPerStage;
          // the tensor-memory buffer is free once the MMAs of the k-stage that used it last
          // (sf_depth k-stages ago) are done: their commit completes a phase of that k-stage's
          // `empty` barrier
          if (need_lag && !ptx::mbar_wait(lag_a, lag_phase, abort_flag, 6)) { ok = false; break; }
          ptx::tc_fence_after_sync();
#pragma unroll
          for (int sub = 0; sub < kSub; ++sub) {
            // 1. atoms of this sub-stage: shared memory -> registers
            const int sub_atoms = atoms - 4 * sub;
            uint32_t ra[16];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v = make_uint4(0u, 0u, 0u, 0u);
              if (j < sub_atoms) v = ptx::ld_shared_v4(src + (sub * 4 + j) * kAtomBytes);
              ra[4 * j] = v.x; ra[4 * j + 1] = v.y; ra[4 * j + 2] = v.z; ra[4 * j + 3] = v.w;
            }
            uint32_t rb[4 * Cfg::kSfbColsPerMma];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
              for (int gi = 0; gi < Cfg::kSfbGroups; ++gi) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (j < sub_atoms)
                  v = ptx::ld_shared_v4(src + kSub * Cfg::kSfaBytes + (gi * kAtomsPerStage + sub * 4 + j) * kAtomBytes);
                const int c = j * Cfg::kSfbColsPerMma + 4 * gi;
                rb[c] = v.x; rb[c + 1] = v.y; rb[c + 2] = v.z; rb[c + 3] = v.w;
              }
            }
            // 2. registers -> the sub-stage's part of this k-stage's tensor-memory buffer
            if (!no_store) {
              ptx::tmem_st_32x32b_x16(taddr + sub * Cfg::kSfColsPerSub, ra);
              if constexpr (Cfg::kSfbGroups == 2) ptx::tmem_st_32x32b_x32(taddr + sub * Cfg::kSfColsPerSub + 16, rb);
              else ptx::tmem_st_32x32b_x16(taddr + sub * Cfg::kSfColsPerSub + 16, rb);
            }
          }
          if (!no_store) ptx::tmem_st_wait();
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (ptx::elect_one()) {
            if constexpr (kTwoCta) ptx::mbar_arrive_cluster(full_t);
            else ptx::mbar_arrive(full_t);
            // the stores above consumed every lane's registers, so the slot's bytes have
            // certainly been read: hand it back to the scale loader
            ptx::mbar_arrive(free_a);
          }
          if (tracing && q == 0 && lane == 0) trace_stamp(p, 3, iter, 1);
        }
        if (need_lag) {
          lag_a += 8;
          if (++lag_stage == kStages) { lag_stage = 0; lag_phase ^= 1; lag_a = empty_u32; }
        }
        src += Cfg::kSfSlotBytes; landed_a += 8; free_a += 8;
        if (++slot == kSfSlots) { slot = 0; slot_phase ^= 1; src = sf_u32 + lane_off; landed_a = sf_landed_u32; free_a = sf_free_u32; }
        ++iter;
        taddr += Cfg::kSfColsPerBuf;
        if (++sfbuf == sf_depth) { sfbuf = 0; taddr = taddr0; }
        full_t += 8;
        if (++stage == kStages) { stage = 0; full_t = full_target_u32; }
      }
    }
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
    uint8_t* stg = staging_base + (warp - kFirstEpilogueWarp) * Cfg::kStagingWarpBytes;
    const uint32_t stg_row = ptx::smem_u32(stg) + lane * 128;
    int acc = 0, tile_iter = 0;
    uint32_t acc_phase = 0;
    for (int task = worker; task < total_tasks; task += num_workers, ++tile_iter) {
      TileCoord t = decode_tile(task, total_mt, n_tiles, p.num_splits, p.raster_m, s_cu_tiles, G);
      const int slab_row = static_cast<int>(cta_rank) * kBlockM + q * 32;   // first row of the slab in the tile
      const int row_in_tile = slab_row + lane;
      const bool row_ok = t.mt * kTileM + row_in_tile < s_rows[t.g];
      const bool slab_full = t.mt * kTileM + slab_row + 32 <= s_rows[t.g];
      const long long out_row = static_cast<long long>(s_row0[t.g]) + t.mt * kTileM + row_in_tile;
      const int col0 = t.nt * BN + half * kWarpCols;
      // A k-split that owns no k-stage (more splits than stages) contributes zeros: the
      // accumulator was never written, so its contents are replaced, not scaled.
      const bool empty_split = (k_stages * t.split) / p.num_splits == (k_stages * (t.split + 1)) / p.num_splits;
      const float alpha = p.group_alpha ? p.group_alpha[t.g] : 1.0f;
      const bool staged = kCanStage && p.tma_store != 0 && slab_full;
      // row coordinate of the slab in the output tensor map (split-K slices are stacked)
      const int map_row = s_row0[t.g] + t.mt * kTileM + slab_row + t.split * p.out_rows_per_split;
      if (!ptx::mbar_wait(acc_full_bar + acc, acc_phase, abort_flag, 4)) break;
      if (warp == kFirstEpilogueWarp && lane == 0) trace_stamp(p, 5, tile_iter, 0);
      ptx::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                             static_cast<uint32_t>(acc * BN + half * kWarpCols);
      auto release_accumulator = [&]() {  // accumulator fully read: hand it back to the MMA warp
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (kTwoCta && !leader) ptx::mbar_arrive_remote(acc_empty_bar + acc, 0);
          else ptx::mbar_arrive(acc_empty_bar + acc);
        }
      };
      // Staged output of 128 bytes per lane (eight 16-byte units in w[0..31]) in two steps, so
      // that the accumulator can be released between them: fill the warp's staging buffer, then
      // hand the 32 x 128-byte box at column `col` to the store engine.
      auto wait_staging_free = [&]() {   // the previous box has left the buffer
        if (lane == 0) ptx::bulk_wait_group_read<0>();
        __syncwarp();
      };
      auto fill_staging = [&](const uint32_t (&w)[32]) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const uint32_t addr = stg_row + (static_cast<uint32_t>(u ^ (lane & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * u]),
                       "r"(w[4 * u + 1]), "r"(w[4 * u + 2]), "r"(w[4 * u + 3])
                       : "memory");
        }
        ptx::fence_proxy_async_smem();
      };
      auto store_staging = [&](int col) {
        __syncwarp();
        if (lane == 0) {
          ptx::tma_store_2d(&tmap_out, stg, col, map_row);
          ptx::bulk_commit_group();
        }
      };

      if constexpr (kSwiGlu) {
        // Accumulator columns 0..127 are the gate, 128..255 the up projection of the same 128
        // intermediate columns. This warp takes 64 of them (4 blocks of 16): both operands are
        // rounded to FP16 first - the values the unfused path would have written and read back -
        // then silu(gate) * up in FP32, quantised per 16 values with one UE4M3 scale.
        const uint32_t g_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN + half * 64);
        uint32_t payload[8];
        uint32_t scale_word = 0;
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          uint32_t gv[32], uv[32];
          ptx::tmem_ld_32x32b_x32(g_addr + pass * 32, gv);
          ptx::tmem_ld_32x32b_x32(g_addr + 128 + pass * 32, uv);
          ptx::tmem_ld_wait();
          if (pass == 1) release_accumulator();
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            float v[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float gf = __half2float(__float2half_rn(__uint_as_float(gv[16 * b + i]) * alpha));
              const float uf = __half2float(__float2half_rn(__uint_as_float(uv[16 * b + i]) * alpha));
              v[i] = __fmul_rn(nvfp4_silu(gf), uf);
            }
            uint32_t lo, hi;
            const uint8_t code = quantize_block16(v, lo, hi);
            payload[(2 * pass + b) * 2] = lo;
            payload[(2 * pass + b) * 2 + 1] = hi;
            scale_word |= static_cast<uint32_t>(code) << (8 * (2 * pass + b));
          }
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
        float* dst = static_cast<float*>(p.out) + t.split * p.out_split_stride + out_row * p.n + col0;
#pragma unroll 1
        for (int c = 0; c < kWarpCols / 32; ++c) {
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(taddr + c * 32, v);
          ptx::tmem_ld_wait();
          if (c == kWarpCols / 32 - 1) release_accumulator();
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
        __half* dst = static_cast<__half*>(p.out) + out_row * p.n + col0;
        constexpr int kChunkCols = kWarpCols >= 64 ? 64 : kWarpCols;     // columns per pass
        constexpr int kChunks = kWarpCols / kChunkCols;
        // Chunk c is converted and put into the staging buffer while the box of chunk c - 1 is
        // still on its way out only after that box has been read; the accumulator is released
        // right after the last TMEM load, before the last box is handed over.
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
        auto direct_store = [&](int c, const uint32_t (&packed)[32]) {
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
          // accumulator goes back to the MMA warp before any output leaves the registers
          uint32_t p0[32], p1[32];
          load_pack(0, p0);
          load_pack(32, p0 + 16);
          load_pack(64, p1);
          load_pack(96, p1 + 16);
          release_accumulator();
          if (warp == kFirstEpilogueWarp && lane == 0) trace_stamp(p, 5, tile_iter, 1);
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
            if (c == kChunks - 1) {
              release_accumulator();
              if (warp == kFirstEpilogueWarp && lane == 0) trace_stamp(p, 5, tile_iter, 1);
            }
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
        if (warp == kFirstEpilogueWarp && lane == 0) trace_stamp(p, 6, tile_iter, 0);
      }
      if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
    }
    // shared memory must outlive the last box
    if (lane == 0) ptx::bulk_wait_group<0>();
    __syncwarp();
  }

  // ---- teardown
  __syncthreads();
  if ((p.debug & 64) && p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long ns;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
    p.trace[((0 * 8 + 7) * 64 + 62) * 2 + 0] = static_cast<unsigned long long>(clock64());
    p.trace[((0 * 8 + 7) * 64 + 62) * 2 + 1] = ns;
  }
  // In a pair neither CTA may leave (or free tensor memory) while the other can still
  // signal its barriers or read its shared memory.
  if constexpr (kTwoCta) ptx::cluster_sync();
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
