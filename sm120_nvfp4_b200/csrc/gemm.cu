// Host launchers and C ABI of the dense / batched / split-K / grouped NVFP4 GEMM.
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include <cuda_fp16.h>

#include "gemm_kernel.cuh"
#include "host_common.hpp"
#include "internal.hpp"

namespace b200 {

__device__ int g_device_error = 0;

int* device_error_word() {
  constexpr int kMaxDevices = 64;
  static int* cache[kMaxDevices] = {};
  static std::mutex mu;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (cache[device] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_device_error) != cudaSuccess) return nullptr;
    cache[device] = static_cast<int*>(ptr);
  }
  return cache[device];
}

std::atomic<long long> g_launch_count{0};

std::atomic<int> g_tile_n_override{0};

// Test hook (b200_nvfp4_set_wait_limit): wait limit of the kernels launched from now on, and a
// one-shot request to withhold one barrier arrival in the next launch.
std::atomic<long long> g_wait_limit{kDefaultWaitLimit};
std::atomic<int> g_withhold_once{0};

namespace {

struct LaunchSpec {
  int num_groups;
  int m_uniform;           // rows per group (dense) - ignored when seqlens != nullptr
  int a_rows_total;        // rows of the A matrix the tensor map covers
  int n, k;
  const void* a;
  const void* b;
  const void* sfa;
  const void* sfb;
  long long sfa_group_stride;
  long long sfb_group_stride;
  int b_group_rows;
  int b_rows_total;
  const int* seqlens;
  const int* cu_seqlens;
  void* out;
  bool out_f32;
  long long out_split_stride;
  const float* group_alpha;
  int num_splits;
  int* tiles_out;
  int* cu_tiles_out;
  int expected_m_tiles;    // estimate used to pick the tile width and the grid
  bool exact_m_tiles;      // expected_m_tiles is exact (dense) rather than a hint (grouped)
  int avg_group_rows;      // rows per group (exact for dense, a hint for grouped)
  int cluster_split = 1;   // 2 / 4: K ranges of a tile on the CTAs of a cluster, reduced on chip (FP16 out)
  int swiglu_inter = 0;    // fused gate/up: intermediate size I (n == 2 * I), else 0
  void* q_out = nullptr;
  void* q_scale = nullptr;
  long long q_scale_group_stride = 0;
  int out_ld = 0;                       // elements between output rows; 0 = n
  long long sfb_atom_rows_total = 0;    // atom rows the B scale map covers; 0 = groups x rows per group
};

template <int BN, bool F32, bool kTwoCta, bool kSwiGlu = false, int kClusterSplit = 1>
int launch_instance(const LaunchSpec& s, const DeviceInfo& dev, cudaStream_t stream) {
  using Cfg = GemmCfg<BN, kTwoCta>;
  auto kernel = nvfp4_gemm_kernel<BN, F32, kTwoCta, kSwiGlu, kClusterSplit>;
  constexpr int kClusterCtas = Cfg::kCtas * kClusterSplit;
  constexpr int kRedBytes = Cfg::red_bytes(kClusterSplit);
  static std::once_flag once[64];
  static cudaError_t attr_status[64];
  std::call_once(once[dev.device], [&] {
    attr_status[dev.device] = cudaFuncSetAttribute(
        kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
  });
  if (attr_status[dev.device] != cudaSuccess) return B200_NVFP4_CUDA_ERROR;

  // Rows of A one load brings in: 128, or the whole (8-row padded) matrix when it is shorter. Only
  // for a single dense problem: groups of a batch or of an expert layout follow each other in
  // memory and tiles address them by row offset.
  int a_box_rows = kBlockM;
  if (!kTwoCta && s.seqlens == nullptr && s.num_groups == 1 && s.m_uniform < kBlockM)
    a_box_rows = (s.m_uniform + 7) / 8 * 8;
  const int a_sub_bytes = a_box_rows * kStageKBytes;
  CUtensorMap tmap_a, tmap_b, tmap_sfa, tmap_sfb;
  const uint64_t row_bytes = static_cast<uint64_t>(s.k) / 2;
  // Scale regions as rank-3 tensors: 128 words of one 512-byte atom, atoms along K, 128-row atom
  // rows (all groups' regions follow each other at a whole number of atom rows). One box = the
  // atoms of a k-stage for one 128-row tile (B: for the one or two scale tiles of a B tile).
  const uint64_t kt = (static_cast<uint64_t>(s.k) + 63) / 64;
  const long long atom_row_bytes = static_cast<long long>(kt) * kAtomBytes;
  const int sfa_group_atom_rows = static_cast<int>(s.sfa_group_stride / atom_row_bytes);
  const int sfb_group_atom_rows = static_cast<int>(s.sfb_group_stride / atom_row_bytes);
  const int b_groups = s.b_group_rows > 0 ? s.b_rows_total / s.b_group_rows : 1;
  if (!encode_tmap_2d_u8(&tmap_a, s.a, static_cast<uint64_t>(s.a_rows_total), row_bytes, a_box_rows,
                         kStageKBytes, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !encode_tmap_2d_u8(&tmap_b, s.b, static_cast<uint64_t>(s.b_rows_total), row_bytes,
                         kSwiGlu ? 128 : Cfg::kBRows, kStageKBytes, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !encode_tmap_sf(&tmap_sfa, s.sfa, kt, static_cast<uint64_t>(s.num_groups) * sfa_group_atom_rows,
                      Cfg::kAtomsPerStage, 1) ||
      !encode_tmap_sf(&tmap_sfb, s.sfb, kt,
                      s.sfb_atom_rows_total > 0 ? static_cast<uint64_t>(s.sfb_atom_rows_total)
                                                : static_cast<uint64_t>(b_groups) * sfb_group_atom_rows,
                      Cfg::kAtomsPerStage, kSwiGlu ? 1 : Cfg::kSfbGroups)) {
    return B200_NVFP4_CUDA_ERROR;
  }

  // Output map for the TMA-store epilogue: boxes of 32 rows x 128 bytes. Split-K slices are
  // stacked along the rows. Tiles of 64 columns and matrices narrower than one box use plain
  // stores only.
  CUtensorMap tmap_out = tmap_a;
  const int box_cols = F32 ? 32 : 64;
  const long long out_rows = static_cast<long long>(s.a_rows_total) * (s.num_splits > 1 ? s.num_splits : 1);
  const bool tma_store = !kSwiGlu && BN >= 128 && s.n >= box_cols && out_rows < 0x7fffffffLL &&
                         encode_tmap_2d_out(&tmap_out, s.out, static_cast<uint64_t>(out_rows),
                                            static_cast<uint64_t>(s.n),
                                            static_cast<uint64_t>(s.out_ld > 0 ? s.out_ld : s.n), F32, 32, box_cols);

  GemmParams p;
  p.tma_store = tma_store ? 1 : 0;
  p.out_rows_per_split = s.num_splits > 1 ? s.a_rows_total : 0;
  p.out_ld = s.out_ld > 0 ? s.out_ld : s.n;
  p.num_groups = s.num_groups;
  p.n = s.n;
  p.k = s.k;
  p.m_uniform = s.m_uniform;
  p.seqlens = s.seqlens;
  p.cu_seqlens = s.cu_seqlens;
  p.sfa_group_atom_rows = sfa_group_atom_rows;
  p.sfb_group_atom_rows = s.b_group_rows > 0 ? sfb_group_atom_rows : 0;
  p.b_group_rows = s.b_group_rows;
  p.out = s.out;
  p.out_split_stride = s.out_split_stride;
  p.group_alpha = s.group_alpha;
  p.num_splits = s.num_splits;
  p.raster_m = kTwoCta ? 8 : 16;
  p.tiles_out = s.tiles_out;
  p.cu_tiles_out = s.cu_tiles_out;
  p.error = device_error_word();
  p.swiglu_inter = s.swiglu_inter;
  p.q_out = static_cast<uint8_t*>(s.q_out);
  p.q_scale = static_cast<uint8_t*>(s.q_scale);
  p.q_scale_group_stride = s.q_scale_group_stride;
  p.a_sub_bytes = a_sub_bytes;
  p.num_stages = Cfg::stages_for(s.num_groups, a_sub_bytes, kRedBytes);
  p.red_bytes = kRedBytes;
  p.wait_limit = g_wait_limit.load(std::memory_order_relaxed);
  p.withhold_first_arrival = g_withhold_once.exchange(0, std::memory_order_relaxed);

  // One persistent worker (a CTA, or a pair of CTAs) per SM (or per SM pair).
  const int n_tiles = kSwiGlu ? s.swiglu_inter / 128 : (s.n + BN - 1) / BN;
  const long long m_tiles = kTwoCta ? (s.expected_m_tiles + 1) / 2 : s.expected_m_tiles;
  long long tasks = m_tiles * n_tiles * (kClusterSplit > 1 ? 1 : s.num_splits);
  int workers = dev.sm_count / kClusterCtas;
  if (kClusterCtas > 1) {
    // Not every SM need be pairable: ask how many pairs can be resident at once, so the
    // persistent grid never queues a pair behind a running one.
    static std::once_flag pair_once[64];
    static int max_pairs[64];
    std::call_once(pair_once[dev.device], [&] {
      cudaLaunchConfig_t probe = {};
      probe.gridDim = dim3(static_cast<unsigned>(dev.sm_count / kClusterCtas * kClusterCtas));
      probe.blockDim = dim3(kGemmThreads);
      probe.dynamicSmemBytes = kSmemBudget;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = kClusterCtas;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      probe.attrs = attr;
      probe.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kernel, &probe) != cudaSuccess || n < 1) n = dev.sm_count / (2 * kClusterCtas);
      max_pairs[dev.device] = n;
    });
    if (workers > max_pairs[dev.device]) workers = max_pairs[dev.device];
  }
  if (s.exact_m_tiles && tasks < workers) workers = static_cast<int>(tasks);
  if (workers < 1) workers = 1;

  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(workers * kClusterCtas));
  config.blockDim = dim3(kGemmThreads);
  config.dynamicSmemBytes = Cfg::smem_bytes(s.num_groups, a_sub_bytes, kRedBytes);
  config.stream = stream;
  cudaLaunchAttribute attrs[1];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = kClusterCtas;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  config.attrs = attrs;
  config.numAttrs = 1;
  const cudaError_t launched = cudaLaunchKernelEx(&config, kernel, tmap_a, tmap_b, tmap_out, tmap_sfa, tmap_sfb, p);
  count_launch();
  const int status = launch_status();
  return launched == cudaSuccess ? status : B200_NVFP4_CUDA_ERROR;
}

// Tile shape. expected_m_tiles counts 128-row tiles.
//   256 x 256 on a CTA pair once there is about a wave of such tiles: tensor-bound shapes,
//     where halving the B traffic per CTA and the deeper pipeline pay;
//   128 x 256 / 128 x 128 / 128 x 64 on single CTAs otherwise - the widest tile that still
//     gives most SMs a task, because skinny problems are bound by streaming B from HBM and
//     need every SM pulling.
// The override (b200_nvfp4_set_tile_n) takes 64 / 128 / 256 for single-CTA tiles and 512 for
// the CTA-pair tile.
constexpr int kPairTileMinRows = 160;

int pick_tile(const LaunchSpec& s, const DeviceInfo& dev) {
  const long long mt = s.expected_m_tiles > 0 ? s.expected_m_tiles : 1;
  const long long splits = s.num_splits;
  auto tasks = [&](int bn) { return mt * ((s.n + bn - 1) / bn) * splits; };
  // a pair tile is 256 rows tall: groups of about 128 rows would leave half of every pair idle
  // (measured on 16 k rows over N = 4096, K = 7168 / N = 7168, K = 2048: a tie at 128 rows per group,
  // the pair tile ahead by 10 - 20 % from 192 rows on)
  const bool tall_groups = s.avg_group_rows >= kPairTileMinRows;
  // the pair tile whenever its pairs occupy (nearly) as many SMs as single 256-column tiles would: the
  // same SMs then work with five operand stages instead of three and two thirds of the L2 traffic
  const long long pair_ctas = 2 * ((mt + 1) / 2) * ((s.n + 255) / 256);
  const long long single_ctas = tasks(256) < dev.sm_count ? tasks(256) : dev.sm_count;
  // ... unless a single dense problem is so small that its pairs cover at most half of the SMs: narrower
  // single-CTA tiles then put more SMs to work (tuner, N = 4096, K = 8192, back to back: M = 256 13.9
  // against 17.2 us, M = 512 16.5 against 18.5; from M = 1024 on the pair tile wins)
  const bool small_dense = s.seqlens == nullptr && s.num_groups == 1 && pair_ctas * 2 <= dev.sm_count;
  if (splits == 1 && tall_groups && !small_dense && pair_ctas * 20 >= single_ctas * 17) return 512;
  if (tasks(256) >= dev.sm_count * 2 / 3) return 256;
  if (tasks(128) >= dev.sm_count * 3 / 4) return 128;
  return 64;
}

// K split over the CTAs of a cluster for a single dense FP16 problem with too few tiles to occupy
// the GPU: the largest of 4 / 2 whose clusters still fit in one wave and leave every CTA at least
// two k-stages. (The caller may have fixed the split: the M = 128 / 256 paths of the dispatcher.)
int pick_cluster_split(const LaunchSpec& s, const DeviceInfo& dev, int tile) {
  if (s.out_f32 || s.num_splits != 1 || s.num_groups != 1 || s.seqlens != nullptr || s.swiglu_inter != 0 ||
      (tile != 64 && tile != 128))
    return 1;
  const long long tasks = static_cast<long long>(s.expected_m_tiles) * ((s.n + tile - 1) / tile);
  const int k_stages = (s.k + (tile == 64 ? 511 : 255)) / (tile == 64 ? 512 : 256);
  for (int split = 4; split >= 2; split /= 2)
    if (tasks * split <= dev.sm_count && k_stages >= 2 * split) return split;
  return 1;
}

// Shape-keyed tile table (b200_nvfp4_tune_set): an entry replaces pick_tile's choice for exactly that
// problem. Key: groups, rows (per problem for dense / batched calls, in total for grouped ones), N,
// K, output type, and whether the row counts come from the device (grouped).
struct TuneKey {
  int groups, rows, n, k, flags;
  bool operator==(const TuneKey& o) const {
    return groups == o.groups && rows == o.rows && n == o.n && k == o.k && flags == o.flags;
  }
};
struct TuneKeyHash {
  size_t operator()(const TuneKey& key) const {
    size_t h = 1469598103934665603ull;
    for (int v : {key.groups, key.rows, key.n, key.k, key.flags}) h = (h ^ static_cast<size_t>(v)) * 1099511628211ull;
    return h;
  }
};
std::mutex g_tune_mutex;
std::unordered_map<TuneKey, int, TuneKeyHash> g_tune_table;
std::atomic<int> g_tune_entries{0};
std::atomic<int> g_last_tile{0};      // tile | cluster split << 16 of the most recent launch_gemm

TuneKey tune_key(int groups, int rows, int n, int k, bool out_f32, bool grouped) {
  return TuneKey{groups, rows, n, k, (out_f32 ? 1 : 0) | (grouped ? 2 : 0)};
}

int tuned_tile(const LaunchSpec& s) {
  if (g_tune_entries.load(std::memory_order_acquire) == 0 || s.swiglu_inter != 0 || s.num_splits != 1) return 0;
  const bool grouped = s.seqlens != nullptr;
  const TuneKey key = tune_key(s.num_groups, grouped ? s.a_rows_total : s.m_uniform, s.n, s.k, s.out_f32, grouped);
  std::lock_guard<std::mutex> lock(g_tune_mutex);
  auto it = g_tune_table.find(key);
  return it == g_tune_table.end() ? 0 : it->second;
}

int launch_gemm(const LaunchSpec& s, cudaStream_t stream, int force_tile = 0) {
  const DeviceInfo& dev = current_device_info();
  if (!dev.ok) return B200_NVFP4_CUDA_ERROR;
  if (!device_supported(dev)) return B200_NVFP4_UNSUPPORTED_DEVICE;
  if (force_tile == 0 && s.cluster_split <= 1) force_tile = tuned_tile(s);
  int tile = force_tile ? force_tile : pick_tile(s, dev);
  if (s.cluster_split > 1 && tile > 128) tile = 128;     // the on-chip reduction is built for 64 / 128 columns
  int split = s.cluster_split > 1 ? s.cluster_split : (s.cluster_split == 1 ? pick_cluster_split(s, dev, tile) : 1);
  // A skinny problem is bound by what one thread can issue per byte of B (four MMAs and eight scale
  // copies per 256 values of K, whatever the tile's width): 128-column tiles with K split four ways
  // move twice the bytes per issued instruction of 64-column tiles split two ways.
  if (!force_tile && s.cluster_split == 1 && tile == 64 && pick_cluster_split(s, dev, 128) == 4) {
    tile = 128;
    split = 4;
  }
  g_last_tile.store(tile | (split << 16), std::memory_order_relaxed);
  if (split > 1) {
    if (tile == 64) return split == 4 ? launch_instance<64, false, false, false, 4>(s, dev, stream)
                                      : launch_instance<64, false, false, false, 2>(s, dev, stream);
    return split == 4 ? launch_instance<128, false, false, false, 4>(s, dev, stream)
                      : launch_instance<128, false, false, false, 2>(s, dev, stream);
  }
  switch (tile) {
    case 512:
      return s.out_f32 ? launch_instance<256, true, true>(s, dev, stream)
                       : launch_instance<256, false, true>(s, dev, stream);
    case 256:
      return s.out_f32 ? launch_instance<256, true, false>(s, dev, stream)
                       : launch_instance<256, false, false>(s, dev, stream);
    case 128:
      return s.out_f32 ? launch_instance<128, true, false>(s, dev, stream)
                       : launch_instance<128, false, false>(s, dev, stream);
    case 64:
      return s.out_f32 ? launch_instance<64, true, false>(s, dev, stream)
                       : launch_instance<64, false, false>(s, dev, stream);
    default:
      return B200_NVFP4_INVALID_ARGUMENT;
  }
}

bool valid_shape(int m, int n, int k) {
  return m > 0 && n > 0 && k > 0 && (k % 32) == 0 && (n % 8) == 0;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Tile-width override for tests and tuning (b200_nvfp4_set_tile_n); 0 = built-in choice.
int env_tile_n() { return g_tile_n_override.load(std::memory_order_relaxed); }

// out[i] = half(sum_s partial[s][i]), summed in split order with FP32 adds
// (reduce_m128_splitk_kernel, src/gemm/specialized/m128_gemm.cu:367-382). numel % 8 == 0.
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, __half* __restrict__ out,
                                     long long numel8, long long split_stride, int splits) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < numel8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8];
    const float4* src = reinterpret_cast<const float4*>(partial + i * 8);
    float4 lo = src[0], hi = src[1];
    acc[0] = lo.x; acc[1] = lo.y; acc[2] = lo.z; acc[3] = lo.w;
    acc[4] = hi.x; acc[5] = hi.y; acc[6] = hi.z; acc[7] = hi.w;
    for (int s = 1; s < splits; ++s) {
      const float4* ps = reinterpret_cast<const float4*>(partial + s * split_stride + i * 8);
      float4 a = ps[0], b = ps[1];
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    uint4 o;
    o.x = pack_half2(acc[0], acc[1]);
    o.y = pack_half2(acc[2], acc[3]);
    o.z = pack_half2(acc[4], acc[5]);
    o.w = pack_half2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + i * 8) = o;
  }
}

}  // namespace

int gemm_dense(int groups, int m, int n, int k, const void* a, const void* b, const void* sfa,
               const void* sfb, void* c, bool out_f32, cudaStream_t stream) {
  if (groups <= 0 || !valid_shape(m, n, k) || a == nullptr || b == nullptr || sfa == nullptr ||
      sfb == nullptr || c == nullptr || groups > kMaxGroups || !aligned16(a) || !aligned16(b) ||
      !aligned16(sfa) || !aligned16(sfb) || !aligned16(c)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  const int skp = scale_k_padded(k);
  LaunchSpec s{};
  s.num_groups = groups;
  s.m_uniform = m;
  s.a_rows_total = groups * m;
  s.n = n;
  s.k = k;
  s.a = a;
  s.b = b;
  s.sfa = sfa;
  s.sfb = sfb;
  s.sfa_group_stride = static_cast<long long>(align_up_int(m, 128)) * skp;
  s.sfb_group_stride = static_cast<long long>(align_up_int(n, 128)) * skp;
  s.b_group_rows = n;
  s.b_rows_total = groups * n;
  s.out = c;
  s.out_f32 = out_f32;
  s.out_split_stride = 0;
  s.num_splits = 1;
  s.expected_m_tiles = groups * ((m + kBlockM - 1) / kBlockM);
  s.exact_m_tiles = true;
  s.avg_group_rows = m;
  return launch_gemm(s, stream, env_tile_n());
}

int gemm_splitk(int m, int n, int k, int split_k, const void* a, const void* b, const void* sfa,
                const void* sfb, void* c_f16, void* workspace, size_t workspace_bytes,
                cudaStream_t stream) {
  if (!valid_shape(m, n, k) || split_k < 1 || split_k > (k + 127) / 128 || a == nullptr ||
      b == nullptr || sfa == nullptr || sfb == nullptr || c_f16 == nullptr ||
      workspace == nullptr || !aligned16(workspace) || !aligned16(a) || !aligned16(b) ||
      !aligned16(sfa) || !aligned16(sfb) || !aligned16(c_f16)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  // split_k <= ceil(K / 128) < 2^24 was checked above; M * N < 2^62, so the byte count is compared by
  // division instead of being formed (it could exceed 64 bits)
  const size_t slice_bytes = static_cast<size_t>(m) * static_cast<size_t>(n) * sizeof(float);
  if (workspace_bytes / slice_bytes < static_cast<size_t>(split_k)) return B200_NVFP4_INSUFFICIENT_WORKSPACE;
  const int skp = scale_k_padded(k);
  LaunchSpec s{};
  s.num_groups = 1;
  s.m_uniform = m;
  s.a_rows_total = m;
  s.n = n;
  s.k = k;
  s.a = a;
  s.b = b;
  s.sfa = sfa;
  s.sfb = sfb;
  s.sfa_group_stride = static_cast<long long>(align_up_int(m, 128)) * skp;
  s.sfb_group_stride = static_cast<long long>(align_up_int(n, 128)) * skp;
  s.b_group_rows = n;
  s.b_rows_total = n;
  s.out = workspace;
  s.out_f32 = true;
  s.out_split_stride = static_cast<long long>(m) * n;
  s.num_splits = split_k;
  s.expected_m_tiles = (m + kBlockM - 1) / kBlockM;
  s.exact_m_tiles = true;
  s.avg_group_rows = m;
  s.cluster_split = 0;
  int status = launch_gemm(s, stream, env_tile_n());
  if (status != B200_NVFP4_SUCCESS) return status;
  const DeviceInfo& dev = current_device_info();
  const long long numel8 = static_cast<long long>(m) * n / 8;
  long long blocks = (numel8 + 255) / 256;
  if (blocks > static_cast<long long>(dev.sm_count) * 8) blocks = static_cast<long long>(dev.sm_count) * 8;
  splitk_reduce_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
      static_cast<const float*>(workspace), static_cast<__half*>(c_f16), numel8,
      static_cast<long long>(m) * n, split_k);
  count_launch();
  return launch_status();
}

// Split-K whose partial tiles never leave the chip: the CTAs of a cluster take the K ranges of
// gemm_splitk (same ranges, same FP32 partial sums, added in the same split order, one rounding to
// FP16 - the result is bit-identical), reduce through distributed shared memory and write C. No
// workspace, one launch. split_k must be 2 or 4.
int gemm_splitk_cluster(int m, int n, int k, int split_k, const void* a, const void* b, const void* sfa,
                        const void* sfb, void* c_f16, cudaStream_t stream) {
  if (!valid_shape(m, n, k) || (split_k != 2 && split_k != 4) || split_k > (k + 127) / 128 || a == nullptr ||
      b == nullptr || sfa == nullptr || sfb == nullptr || c_f16 == nullptr || !aligned16(a) || !aligned16(b) ||
      !aligned16(sfa) || !aligned16(sfb) || !aligned16(c_f16)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  const int skp = scale_k_padded(k);
  LaunchSpec s{};
  s.num_groups = 1;
  s.m_uniform = m;
  s.a_rows_total = m;
  s.n = n;
  s.k = k;
  s.a = a;
  s.b = b;
  s.sfa = sfa;
  s.sfb = sfb;
  s.sfa_group_stride = static_cast<long long>(align_up_int(m, 128)) * skp;
  s.sfb_group_stride = static_cast<long long>(align_up_int(n, 128)) * skp;
  s.b_group_rows = n;
  s.b_rows_total = n;
  s.out = c_f16;
  s.out_f32 = false;
  s.num_splits = 1;
  s.expected_m_tiles = (m + kBlockM - 1) / kBlockM;
  s.exact_m_tiles = true;
  s.avg_group_rows = m;
  s.cluster_split = split_k;
  // 128-column tiles unless that leaves most SMs without a cluster
  const DeviceInfo& dev = current_device_info();
  const long long tasks128 = static_cast<long long>(s.expected_m_tiles) * ((n + 127) / 128);
  int tile = env_tile_n();
  if (tile != 64 && tile != 128) tile = (dev.ok && tasks128 * split_k * 2 <= dev.sm_count) ? 64 : 128;
  return launch_gemm(s, stream, tile);
}

int gemm_grouped(void* y, const void* x, const void* w, const void* seqlens,
                 const void* cu_seqlens, const void* x_scale, const void* w_scale, void* tiles,
                 void* cu_tiles, int num_group, int m, int n, int k, int m_scale_pad,
                 int num_seq_per_group_avg, const float* group_alpha, cudaStream_t stream,
                 int col_start, int col_count) {
  // Column window: the launch computes y[:, col_start : col_start + col_count) of the full
  // [m, n] product; everything else about the call (w, w_scale, y as whole arrays) stays.
  if (col_count == 0) col_count = n - col_start;
  if (col_start < 0 || (col_start % 128) != 0 || col_count <= 0 || col_start > n - col_count ||
      (col_start + col_count < n && (col_count % 128) != 0)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  if (num_group <= 0 || num_group > kMaxGroups || !valid_shape(m, n, k) || y == nullptr ||
      x == nullptr || w == nullptr || seqlens == nullptr || cu_seqlens == nullptr ||
      x_scale == nullptr || w_scale == nullptr || m_scale_pad < 128 || (m_scale_pad % 128) != 0 ||
      !aligned16(y) || !aligned16(x) || !aligned16(w) || !aligned16(x_scale) ||
      !aligned16(w_scale)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  const int skp = scale_k_padded(k);
  LaunchSpec s{};
  s.num_groups = num_group;
  s.m_uniform = 0;
  s.a_rows_total = m;
  s.n = col_count;
  s.k = k;
  s.a = x;
  s.b = static_cast<const uint8_t*>(w) + static_cast<long long>(col_start) * (k / 2);
  s.sfa = x_scale;
  s.sfb = static_cast<const uint8_t*>(w_scale) + static_cast<long long>(col_start) * skp;
  s.sfa_group_stride = static_cast<long long>(m_scale_pad) * skp;
  s.sfb_group_stride = static_cast<long long>(align_up_int(n, 128)) * skp;
  s.b_group_rows = n;
  s.b_rows_total = num_group * n - col_start;
  s.sfb_atom_rows_total = static_cast<long long>(num_group) * (align_up_int(n, 128) / 128) - col_start / 128;
  s.seqlens = static_cast<const int*>(seqlens);
  s.cu_seqlens = static_cast<const int*>(cu_seqlens);
  s.out = static_cast<__half*>(y) + col_start;
  s.out_ld = n;
  s.out_f32 = false;
  s.num_splits = 1;
  s.group_alpha = group_alpha;
  s.tiles_out = static_cast<int*>(tiles);
  s.cu_tiles_out = static_cast<int*>(cu_tiles);
  // Row counts live on the device; estimate the m-tiles for the tile-width heuristic only.
  int avg = num_seq_per_group_avg > 0 ? num_seq_per_group_avg : (m + num_group - 1) / num_group;
  long long est = static_cast<long long>(num_group) * ((avg + kBlockM - 1) / kBlockM);
  long long upper = static_cast<long long>(m) / kBlockM + num_group;
  if (est > upper) est = upper;
  if (est < 1) est = 1;
  s.expected_m_tiles = static_cast<int>(est);
  s.exact_m_tiles = false;
  s.avg_group_rows = avg;
  s.cluster_split = 0;
  return launch_gemm(s, stream, env_tile_n());
}

// Gate/up grouped GEMM with the SiLU * up + NVFP4 quantisation in its epilogue: w is
// [G, 2I, K/2] (gate rows, then up rows), the result is what moe_act_mul_and_quant would
// make of the FP16 product - packed [m, I/2] and per-group scale regions of q_scale_m_pad rows -
// bit for bit. Returns B200_NVFP4_CUTLASS_NOT_SUPPORTED for shapes the fused tile does not
// cover (I not a multiple of 128); the caller then runs the two separate steps.
int gemm_grouped_swiglu(void* q_out, void* q_scale, const void* x, const void* w, const void* seqlens,
                        const void* cu_seqlens, const void* x_scale, const void* w_scale, void* tiles,
                        void* cu_tiles, int num_group, int m, int inter, int k, int m_scale_pad,
                        int q_scale_m_pad, int num_seq_per_group_avg, cudaStream_t stream) {
  if (inter <= 0 || (inter % 128) != 0) return B200_NVFP4_CUTLASS_NOT_SUPPORTED;
  const int n = 2 * inter;
  if (num_group <= 0 || num_group > kMaxGroups || !valid_shape(m, n, k) || q_out == nullptr ||
      q_scale == nullptr || x == nullptr || w == nullptr || seqlens == nullptr ||
      cu_seqlens == nullptr || x_scale == nullptr || w_scale == nullptr || m_scale_pad < 128 ||
      (m_scale_pad % 128) != 0 || q_scale_m_pad < 128 || (q_scale_m_pad % 128) != 0 ||
      !aligned16(q_out) || !aligned16(q_scale) || !aligned16(x) || !aligned16(w) ||
      !aligned16(x_scale) || !aligned16(w_scale)) {
    return B200_NVFP4_INVALID_ARGUMENT;
  }
  const DeviceInfo& dev = current_device_info();
  if (!dev.ok) return B200_NVFP4_CUDA_ERROR;
  if (!device_supported(dev)) return B200_NVFP4_UNSUPPORTED_DEVICE;
  const int skp = scale_k_padded(k);
  LaunchSpec s{};
  s.num_groups = num_group;
  s.m_uniform = 0;
  s.a_rows_total = m;
  s.n = n;
  s.k = k;
  s.a = x;
  s.b = w;
  s.sfa = x_scale;
  s.sfb = w_scale;
  s.sfa_group_stride = static_cast<long long>(m_scale_pad) * skp;
  s.sfb_group_stride = static_cast<long long>(align_up_int(n, 128)) * skp;
  s.b_group_rows = n;
  s.b_rows_total = num_group * n;
  s.seqlens = static_cast<const int*>(seqlens);
  s.cu_seqlens = static_cast<const int*>(cu_seqlens);
  s.out = q_out;   // not written as a matrix; kept non-null for the common checks
  s.out_f32 = false;
  s.num_splits = 1;
  s.tiles_out = static_cast<int*>(tiles);
  s.cu_tiles_out = static_cast<int*>(cu_tiles);
  int avg = num_seq_per_group_avg > 0 ? num_seq_per_group_avg : (m + num_group - 1) / num_group;
  long long est = static_cast<long long>(num_group) * ((avg + kBlockM - 1) / kBlockM);
  const long long upper = static_cast<long long>(m) / kBlockM + num_group;
  if (est > upper) est = upper;
  if (est < 1) est = 1;
  s.expected_m_tiles = static_cast<int>(est);
  s.exact_m_tiles = false;
  s.avg_group_rows = avg;
  s.swiglu_inter = inter;
  s.q_out = q_out;
  s.q_scale = q_scale;
  s.q_scale_group_stride = static_cast<long long>(q_scale_m_pad) * scale_k_padded(inter);
  // tall groups on CTA pairs, short ones on single CTAs: the rule of the plain grouped GEMM
  const int forced = env_tile_n();
  const bool pair = forced ? forced == 512
                           : (avg >= kPairTileMinRows && ((est + 1) / 2) * (inter / 128) >= dev.sm_count / 2);
  return pair ? launch_instance<256, false, true, true>(s, dev, stream)
              : launch_instance<256, false, false, true>(s, dev, stream);
}

}  // namespace b200

// --------------------------------------------------------------------------- C ABI

extern "C" {

const char* b200_nvfp4_status_string(int status) {
  switch (status) {
    case B200_NVFP4_SUCCESS: return "success";
    case B200_NVFP4_INVALID_ARGUMENT: return "invalid argument or unsupported alignment";
    case B200_NVFP4_UNSUPPORTED_DEVICE: return "current device is not SM100 (B200)";
    case B200_NVFP4_INSUFFICIENT_WORKSPACE: return "workspace is null or too small";
    case B200_NVFP4_CUTLASS_NOT_SUPPORTED: return "CUTLASS cannot implement this problem shape/alignment";
    case B200_NVFP4_CUTLASS_ERROR: return "CUTLASS initialize or launch failed";
    case B200_NVFP4_CUDA_ERROR: return "CUDA runtime error";
  }
  return "unknown status";
}

const char* b200_nvfp4_gemm_path_string(int path) {
  switch (path) {
    case B200_NVFP4_PATH_GENERIC: return "generic_cute";
    case B200_NVFP4_PATH_M128_SPLITK4: return "m128_splitk4";
    case B200_NVFP4_PATH_M256_SPLITK2: return "m256_splitk2";
  }
  return "unknown";
}

int b200_nvfp4_gemm_path(int m, int n, int k) {
  const bool shape_ok = n > 0 && k > 0 && (k % 32) == 0 && (n % 8) == 0;
  const int tiles_k = (k + 127) / 128;
  if (m == 128 && shape_ok && 4 <= tiles_k) return B200_NVFP4_PATH_M128_SPLITK4;
  if (m == 256 && shape_ok && 2 <= tiles_k) return B200_NVFP4_PATH_M256_SPLITK2;
  return B200_NVFP4_PATH_GENERIC;
}

size_t b200_nvfp4_gemm_workspace_bytes(int m, int n, int k) {
  switch (b200_nvfp4_gemm_path(m, n, k)) {
    case B200_NVFP4_PATH_M128_SPLITK4: return static_cast<size_t>(4) * m * n * sizeof(float);
    case B200_NVFP4_PATH_M256_SPLITK2: return static_cast<size_t>(2) * m * n * sizeof(float);
    default: return 0;
  }
}

int b200_nvfp4_gemm(int groups, int m, int n, int k, const void* a, const void* b, const void* sfa,
                    const void* sfb, void* c, int out_is_f32, b200_stream_t stream) {
  return b200::gemm_dense(groups, m, n, k, a, b, sfa, sfb, c, out_is_f32 != 0,
                          static_cast<cudaStream_t>(stream));
}

int b200_nvfp4_gemm_splitk(int m, int n, int k, int split_k, const void* a, const void* b,
                           const void* sfa, const void* sfb, void* c_f16, void* workspace,
                           size_t workspace_bytes, b200_stream_t stream) {
  return b200::gemm_splitk(m, n, k, split_k, a, b, sfa, sfb, c_f16, workspace, workspace_bytes,
                           static_cast<cudaStream_t>(stream));
}

int b200_nvfp4_gemm_splitk_cluster(int m, int n, int k, int split_k, const void* a, const void* b,
                                   const void* sfa, const void* sfb, void* c_f16, b200_stream_t stream) {
  return b200::gemm_splitk_cluster(m, n, k, split_k, a, b, sfa, sfb, c_f16, static_cast<cudaStream_t>(stream));
}

int b200_nvfp4_gemm_auto(int m, int n, int k, const void* a, const void* b, const void* sfa,
                         const void* sfb, void* c_f16, void* workspace, size_t workspace_bytes,
                         b200_stream_t stream) {
  const int path = b200_nvfp4_gemm_path(m, n, k);
  const size_t required = b200_nvfp4_gemm_workspace_bytes(m, n, k);
  if (required != 0 && (workspace == nullptr || workspace_bytes < required))
    return B200_NVFP4_INSUFFICIENT_WORKSPACE;
  // The reference's M = 128 / 256 paths: split-K 4 / 2 with the partial sums added in split order.
  // The workspace the reference ABI asks for is still required (same status codes) but not used:
  // the partial tiles are reduced on chip (b200_nvfp4_gemm_splitk_cluster), with the bits
  // b200_nvfp4_gemm_splitk gives on the same operands.
  switch (path) {
    case B200_NVFP4_PATH_M128_SPLITK4:
      return b200::gemm_splitk_cluster(m, n, k, 4, a, b, sfa, sfb, c_f16, static_cast<cudaStream_t>(stream));
    case B200_NVFP4_PATH_M256_SPLITK2:
      return b200::gemm_splitk_cluster(m, n, k, 2, a, b, sfa, sfb, c_f16, static_cast<cudaStream_t>(stream));
    default:
      return b200_nvfp4_gemm(1, m, n, k, a, b, sfa, sfb, c_f16, 0, stream);
  }
}

int b200_nvfp4_grouped_gemm(void* y, const void* x, const void* w, const void* seqlens,
                            const void* cu_seqlens, const void* x_scale, const void* w_scale,
                            void* tmas, void* tiles, void* cu_tiles, int num_group, int m, int n,
                            int k, int m_scale_pad, int num_seq_per_group_avg, int update_tma,
                            const float* group_alpha, b200_stream_t stream) {
  (void)tmas;
  (void)update_tma;
  return b200::gemm_grouped(y, x, w, seqlens, cu_seqlens, x_scale, w_scale, tiles, cu_tiles,
                            num_group, m, n, k, m_scale_pad, num_seq_per_group_avg, group_alpha,
                            static_cast<cudaStream_t>(stream), 0, 0);
}

int b200_nvfp4_grouped_gemm_columns(void* y, const void* x, const void* w, const void* seqlens,
                                    const void* cu_seqlens, const void* x_scale, const void* w_scale,
                                    int num_group, int m, int n, int k, int m_scale_pad,
                                    int num_seq_per_group_avg, const float* group_alpha, int col_start,
                                    int col_count, b200_stream_t stream) {
  if (col_count <= 0) return B200_NVFP4_INVALID_ARGUMENT;
  return b200::gemm_grouped(y, x, w, seqlens, cu_seqlens, x_scale, w_scale, nullptr, nullptr, num_group, m, n,
                            k, m_scale_pad, num_seq_per_group_avg, group_alpha,
                            static_cast<cudaStream_t>(stream), col_start, col_count);
}

int b200_nvfp4_device_error(int* code) {
  int* word = b200::device_error_word();
  if (word == nullptr || code == nullptr) return B200_NVFP4_CUDA_ERROR;
  int value = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return B200_NVFP4_CUDA_ERROR;
  if (cudaMemcpy(&value, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
    return B200_NVFP4_CUDA_ERROR;
  if (value != 0) {
    int zero = 0;
    if (cudaMemcpy(word, &zero, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess)
      return B200_NVFP4_CUDA_ERROR;
  }
  *code = value;
  return B200_NVFP4_SUCCESS;
}

int b200_nvfp4_set_tile_n(int tile_n) {
  if (tile_n != 0 && tile_n != 64 && tile_n != 128 && tile_n != 256 && tile_n != 512)
    return B200_NVFP4_INVALID_ARGUMENT;
  b200::g_tile_n_override.store(tile_n, std::memory_order_relaxed);
  return B200_NVFP4_SUCCESS;
}

int b200_nvfp4_tune_set(int groups, int rows, int n, int k, int out_f32, int grouped, int tile_n) {
  if (groups <= 0 || rows <= 0 || n <= 0 || k <= 0 ||
      (tile_n != 0 && tile_n != 64 && tile_n != 128 && tile_n != 256 && tile_n != 512))
    return B200_NVFP4_INVALID_ARGUMENT;
  const b200::TuneKey key = b200::tune_key(groups, rows, n, k, out_f32 != 0, grouped != 0);
  std::lock_guard<std::mutex> lock(b200::g_tune_mutex);
  if (tile_n == 0) b200::g_tune_table.erase(key);
  else b200::g_tune_table[key] = tile_n;
  b200::g_tune_entries.store(static_cast<int>(b200::g_tune_table.size()), std::memory_order_release);
  return B200_NVFP4_SUCCESS;
}

int b200_nvfp4_tune_get(int groups, int rows, int n, int k, int out_f32, int grouped) {
  const b200::TuneKey key = b200::tune_key(groups, rows, n, k, out_f32 != 0, grouped != 0);
  std::lock_guard<std::mutex> lock(b200::g_tune_mutex);
  auto it = b200::g_tune_table.find(key);
  return it == b200::g_tune_table.end() ? 0 : it->second;
}

int b200_nvfp4_last_launch_tile(void) { return b200::g_last_tile.load(std::memory_order_relaxed); }

void b200_nvfp4_tune_clear(void) {
  std::lock_guard<std::mutex> lock(b200::g_tune_mutex);
  b200::g_tune_table.clear();
  b200::g_tune_entries.store(0, std::memory_order_release);
}

int b200_nvfp4_set_wait_limit(long long limit_cycles, int withhold_one_arrival) {
  if (limit_cycles < 0) return B200_NVFP4_INVALID_ARGUMENT;
  b200::g_wait_limit.store(limit_cycles > 0 ? limit_cycles : b200::kDefaultWaitLimit, std::memory_order_relaxed);
  b200::g_withhold_once.store(withhold_one_arrival != 0 ? 1 : 0, std::memory_order_relaxed);
  return B200_NVFP4_SUCCESS;
}

long long b200_nvfp4_launch_count(void) {
  return b200::g_launch_count.load(std::memory_order_relaxed);
}

}  // extern "C"
