// Inline-PTX wrappers for the sm_100a features the GEMM kernel uses: mbarrier, TMA (tiled loads
// and stores), tensor memory (TMEM) allocation, tcgen05.mma / cp / ld / commit, and the UMMA
// descriptors. Shared-memory operands are 32-bit shared-window addresses throughout: the role
// loops of the kernel are chains of dependent scalar instructions, and a ring position that
// advances by a 32-bit add costs less than a generic pointer that needs 64-bit arithmetic and a
// conversion before every use.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace b200 {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// True in exactly one (always the same) lane of a fully active warp. Code that issues
// single-thread instructions (TMA, tcgen05.mma, tcgen05.commit) keeps the whole warp in
// uniform control flow and wraps only the instruction in `if (elect_one())`, so the compiler
// can hold addresses and descriptors in uniform registers instead of moving them there from
// one lane's registers before every instruction.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, UMMA).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// Arrive on a barrier given by its shared::cluster address (this or another CTA of the cluster).
// Default (CTA-scope release) semantics: a cluster-scope release costs the arriving thread more
// than a microsecond, and what these arrivals order - tensor-memory traffic - is ordered by the
// tcgen05 fences on both sides.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking probe of the same condition (never suspends the thread).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Orders this thread's earlier accesses (including stores into other CTAs' shared memory) before
// its later ones at cluster scope.
__device__ __forceinline__ void fence_acq_rel_cluster() {
  asm volatile("fence.acq_rel.cluster;" ::: "memory");
}

// Arrival on a barrier of another CTA that publishes this thread's earlier stores into that CTA's
// shared memory (release at cluster scope): the counterpart of mbar_wait_cluster.
__device__ __forceinline__ void mbar_arrive_release_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait_acquire_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. Every wait in the kernel gives up after `limit` clock cycles (about a second by
// default), records `code` in *abort_flag (shared) and returns false, so a protocol bug can never
// hang the GPU. Once the flag is set all later waits return at once. The common case - the phase
// is already complete - is a single non-blocking probe, which returns in less than half the time
// of try_wait.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code,
                                          long long limit) {
  if (mbar_test_wait(bar, parity)) return true;
  long long start = clock64();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 255u) == 0) {
      if (*abort_flag != 0) return false;
      if (clock64() - start > limit) {
        atomicCAS(const_cast<int*>(abort_flag), 0, code);
        return false;
      }
    }
  }
}

// The same bounded wait with acquire semantics at cluster scope: what other CTAs of the cluster
// stored into this CTA's shared memory before their releasing arrivals is visible afterwards.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code,
                                                  long long limit) {
  long long start = clock64();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait_acquire_cluster(bar, parity)) return true;
    if ((++spins & 255u) == 0) {
      if (*abort_flag != 0) return false;
      if (clock64() - start > limit) {
        atomicCAS(const_cast<int*>(abort_flag), 0, code);
        return false;
      }
    }
  }
}

// --------------------------------------------------------------------- TMA

__device__ __forceinline__ void prefetch_tensormap(const void* desc) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(desc)) : "memory");
}

// 2-D tiled load global -> shared, completion counted in bytes on `bar`.
// c0 (innermost coordinate) times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const void* desc, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// Same load issued by a CTA of a pair (cta_group::2): the data goes to this CTA's shared
// memory, the completion bytes to the mbarrier at shared::cluster address `bar_cluster_addr`,
// which may belong to the other CTA of the pair. Each CTA loads its own tile.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const void* desc, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}

// 3-D variants (scale-factor atoms: word inside the atom, atom along K, 128-row atom row).
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const void* desc, uint32_t bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair(uint32_t smem_dst, const void* desc, uint32_t bar_cluster_addr,
                                                 int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// 2-D tiled store shared -> global (bulk async-group completion).
__device__ __forceinline__ void tma_store_2d(const void* desc, uint32_t smem_src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::
                   "l"(reinterpret_cast<uint64_t>(desc)),
               "r"(smem_src), "r"(c0), "r"(c1)
               : "memory");
}

__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ------------------------------------------------------------ tensor memory

// The tcgen05 wrappers below take the CTA-group size as a template argument: 1 = the
// instruction acts on this CTA only, 2 = it acts on both CTAs of a pair (a cluster of two
// CTAs on one TPC that issue one 256-row MMA together).

// Whole-warp call. ncols: power of two in [32, 512]. The base address is written to shared memory
// at `smem_out`. With kCtas == 2 the same warp of both CTAs must call it.
template <int kCtas>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_out, uint32_t ncols) {
  if constexpr (kCtas == 2)
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_out), "r"(ncols) : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_out), "r"(ncols) : "memory");
}

template <int kCtas>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (kCtas == 2)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

template <int kCtas>
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t ncols) {
  if constexpr (kCtas == 2)
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(ncols) : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Arrives (count 1) on `bar` once all tcgen05 operations this thread issued so far are done.
// kCtas == 2: the arrival is delivered to the barrier at the same shared-memory offset in
// every CTA of the pair selected by cta_mask (bit i = CTA rank i).
template <int kCtas>
__device__ __forceinline__ void tc_commit(uint32_t bar, uint16_t cta_mask = 1) {
  if constexpr (kCtas == 2)
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
        "[%0], %1;" ::"r"(bar), "h"(cta_mask)
        : "memory");
  else
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Shared -> tensor memory copy of one scale-factor atom: 32 rows x 128 bits, replicated into the
// four 32-lane quarters (the form the block-scaled MMA wants). The source is named by a
// shared-memory matrix descriptor given as its two 32-bit halves. With kCtas == 2 each CTA of the
// pair copies from its own shared memory (same offset) into its own tensor memory. The copy is
// ordered with the tcgen05.mma instructions the same thread issues before and after it.
template <int kCtas>
__device__ __forceinline__ void tc_cp_32x128b_warpx4(uint32_t tmem_dst, uint32_t desc_lo, uint32_t desc_hi) {
  if constexpr (kCtas == 2)
    asm volatile(
        "{\n\t.reg .b64 d;\n\t"
        "mov.b64 d, {%1, %2};\n\t"
        "tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], d;\n\t}" ::"r"(tmem_dst), "r"(desc_lo), "r"(desc_hi)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .b64 d;\n\t"
        "mov.b64 d, {%1, %2};\n\t"
        "tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], d;\n\t}" ::"r"(tmem_dst), "r"(desc_lo), "r"(desc_hi)
        : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T with E2M1 operands and one UE4M3 scale per 16 K-elements
// (K = 64 per instruction). accumulate == 0 overwrites D. kCtas == 2: one 256 x N MMA over
// the pair; each CTA supplies 128 rows of A and N/2 rows of B from its own shared memory
// (same offsets in both) and accumulates its 128 rows in its own TMEM. The shared-memory
// descriptors are given as their low words (start address and leading-dimension offset) plus one
// high word common to both (stride offset, version, swizzle): advancing along K or to the next
// stage is a 32-bit add on the low word.
template <int kCtas>
__device__ __forceinline__ void tc_mma_nvfp4(uint32_t tmem_d, uint32_t desc_a_lo, uint32_t desc_b_lo,
                                             uint32_t desc_hi, uint32_t idesc, uint32_t tmem_sfa,
                                             uint32_t tmem_sfb, uint32_t accumulate) {
  if constexpr (kCtas == 2)
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], da, db, %4, [%6], [%7], "
        "p;\n\t}" ::"r"(tmem_d),
        "r"(desc_a_lo), "r"(desc_b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], da, db, %4, [%6], [%7], "
        "p;\n\t}" ::"r"(tmem_d),
        "r"(desc_a_lo), "r"(desc_b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives lane (base_lane + t).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// Same, 8 consecutive columns.
// (The destination registers hold the data only after tmem_ld_wait(): nothing may read or copy
// them in between, so callers that batch several loads pass the final destination.)
__device__ __forceinline__ void tmem_ld_32x32b_x8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ------------------------------------------------------------------ clusters

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// The two halves of the cluster barrier: every thread of every CTA arrives once and waits once per
// phase, not necessarily at the same place in the program.
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
// Arrival without a release of this thread's earlier writes: enough after set-up, where the only
// writes the partners must see - the mbarrier initialisations - were published by
// fence_barrier_init(), and far cheaper than a cluster-scope release.
__device__ __forceinline__ void cluster_arrive_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Named CTA barriers (ids 1..15; id 0 is __syncthreads): `count` threads take part, each either
// waits for the others (sync) or only reports (arrive). Whole warps only.
__device__ __forceinline__ void named_barrier_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_barrier_arrive(int id, int count) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// Barrier over all threads of all CTAs in the cluster (release / acquire).
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// shared::cluster address of the object at shared-memory address `smem_addr` of this CTA, seen in
// the CTA with rank `cta_rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta_rank));
  return r;
}

// Stores / loads through a shared::cluster address (distributed shared memory).
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}

// Asynchronous 16-byte store into the shared memory of a CTA of this cluster; on completion it adds
// 16 to the transaction count of the mbarrier `bar_cluster_addr` (same CTA as the data), so the
// receiver's wait on that barrier covers the data: no fence or separate arrival by the sender.
__device__ __forceinline__ void st_async_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d,
                                            uint32_t bar_cluster_addr) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(addr),
               "r"(a), "r"(b), "r"(c), "r"(d), "r"(bar_cluster_addr)
               : "memory");
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// ------------------------------------------------------------- descriptors
//
// Shared-memory matrix descriptor (64 bit) for tcgen05.mma / tcgen05.cp:
//   [0,14)  start address >> 4          [16,30) leading-dimension byte offset >> 4
//   [32,46) stride-dimension byte offset >> 4   [46,48) descriptor version (1 on sm_100)
//   [61,64) swizzle mode: 0 none, 2 = 128-byte, 4 = 64-byte, 6 = 32-byte

// K-major operand tile whose rows are 128 bytes (256 E2M1 values) written by TMA with the
// 128-byte swizzle: 8-row groups are 1024 bytes apart (leading-dimension offset 16 bytes).
constexpr uint32_t kKmajorSw128LboBits = (16u >> 4) << 16;
__device__ __forceinline__ uint32_t kmajor_sw128_desc_lo(uint32_t smem_addr) {
  return ((smem_addr >> 4) & 0x3fffu) | kKmajorSw128LboBits;
}
constexpr uint32_t kKmajorSw128DescHi = ((1024u >> 4) & 0x3fffu) | (1u << 14) | (2u << 29);

// One 512-byte scale-factor atom: 32 rows x 16 bytes, unswizzled, 8-row groups 128 bytes apart.
constexpr uint32_t kSfAtomDescHi = ((128u >> 4) & 0x3fffu) | (1u << 14);

// Instruction descriptor of the block-scaled MMA (kind::mxf4nvf4): E2M1 x E2M1, UE4M3 scales,
// both operands K-major, FP32 accumulate, M x N x 64.
//   [7,10) A format (1 = E2M1)   [10,13) B format   [15] A major   [16] B major
//   [17,23) N >> 3   [23] scale format (0 = UE4M3)   [24,29) M >> 4
//   [4,6) / [29,31) scale-factor byte ids (0 with four scales per row per instruction)
__host__ __device__ constexpr uint32_t make_idesc_nvfp4(int m, int n) {  // m = 128, or 256 for a CTA pair
  return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

}  // namespace ptx
}  // namespace b200
