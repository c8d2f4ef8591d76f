// Exercises the C++ API (namespace sm120_nvfp4) the way a caller of the reference library
// uses it: only the three public headers, cudart for memory. Plays the part of the
// reference's tests/cpp/test_gemm.cu (dispatcher table :95-103, known-answer GEMM, status
// codes) and of the uniform-data MoE case of tests/python/test_fused_moe.py:55-101.
//
//   api_check host     checks that need no GPU: dispatcher table, strings, sizes, argument errors
//   api_check device   known-answer runs on the current CUDA device
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include "sm120_nvfp4/fused_moe.hpp"
#include "sm120_nvfp4/gemm.hpp"
#include "sm120_nvfp4/grouped_gemm.hpp"

namespace api = sm120_nvfp4;

static int g_failures = 0;
#define EXPECT(cond)                                                            \
  do {                                                                          \
    if (!(cond)) {                                                              \
      std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond);               \
      ++g_failures;                                                             \
    }                                                                           \
  } while (0)

static void cuda_ok(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

template <typename T>
struct DeviceBuffer {
  T* ptr = nullptr;
  std::size_t count = 0;
  explicit DeviceBuffer(std::size_t n) : count(n) { cuda_ok(cudaMalloc(reinterpret_cast<void**>(&ptr), (n ? n : 1) * sizeof(T)), "cudaMalloc"); }
  ~DeviceBuffer() { cudaFree(ptr); }
  void fill_bytes(int value) { cuda_ok(cudaMemset(ptr, value, count * sizeof(T)), "cudaMemset"); }
  void upload(const std::vector<T>& h) { cuda_ok(cudaMemcpy(ptr, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice), "upload"); }
  std::vector<T> download() const {
    std::vector<T> h(count);
    cuda_ok(cudaMemcpy(h.data(), ptr, count * sizeof(T), cudaMemcpyDeviceToHost), "download");
    return h;
  }
};

static int host_checks() {
  using api::GemmStatus;
  using api::Nvfp4GemmPath;
  struct Row { int m, n, k; Nvfp4GemmPath path; std::size_t workspace; };
  const Row table[] = {
      {16, 4096, 8192, Nvfp4GemmPath::kGenericCute, 0},
      {128, 4096, 8192, Nvfp4GemmPath::kM128SplitK4, std::size_t{4} * 128 * 4096 * 4},
      {256, 4096, 8192, Nvfp4GemmPath::kM256SplitK2, std::size_t{2} * 256 * 4096 * 4},
      {128, 128, 128, Nvfp4GemmPath::kGenericCute, 0},   // one 128-wide k-tile cannot be split in four
      {256, 4096, 136, Nvfp4GemmPath::kGenericCute, 0},  // K % 32 != 0
  };
  for (const Row& r : table) {
    EXPECT(api::nvfp4_gemm_path_sm120(r.m, r.n, r.k) == r.path);
    EXPECT(api::nvfp4_gemm_workspace_size_sm120(r.m, r.n, r.k) == r.workspace);
  }
  EXPECT(std::strcmp(api::nvfp4_gemm_path_string(Nvfp4GemmPath::kM128SplitK4), "m128_splitk4") == 0);
  EXPECT(std::strcmp(api::gemm_status_string(GemmStatus::kSuccess), "success") == 0);
  EXPECT(static_cast<int>(GemmStatus::kCudaError) == 6);
  EXPECT(api::scale_k_padded(8192) == 512 && api::scale_k_padded(7168) == 448 && api::scale_k_padded(2048) == 128);
  EXPECT(api::scale_a_elements(16, 4096, 8192) == std::size_t{128} * 512);
  EXPECT(api::scale_b_elements(16, 4096, 8192) == std::size_t{4096} * 512);
  EXPECT(api::packed_fp4_bytes(16, 8192) == std::size_t{16} * 4096);
  // argument errors are reported before any device is touched
  half* none = nullptr;
  EXPECT(api::nvfp4_cute_gemm_sm120(16, 128, 128, nullptr, nullptr, nullptr, nullptr, none) == GemmStatus::kInvalidArgument);
  int dummy = 0;
  EXPECT(api::nvfp4_cute_gemm_sm120(16, 128, 100, &dummy, &dummy, &dummy, &dummy, reinterpret_cast<half*>(&dummy)) ==
         GemmStatus::kInvalidArgument);
  EXPECT(api::nvfp4_gemm_sm120(128, 4096, 8192, reinterpret_cast<void*>(16), reinterpret_cast<void*>(16),
                              reinterpret_cast<void*>(16), reinterpret_cast<void*>(16),
                              reinterpret_cast<half*>(16), nullptr, 0) == GemmStatus::kInsufficientWorkspace);
  EXPECT(api::fused_moe::expert_moe_nvfp4_workspace_size(512, 7168, 2048, 32, 128) > std::size_t{512} * 4096 * 2);
  bool threw = false;
  try {
    api::fused_moe::expert_moe_nvfp4_async(&dummy, &dummy, &dummy, &dummy, &dummy, &dummy, &dummy, &dummy, &dummy,
                                          nullptr, 0, 512, 7168, 2048, 32, 128, nullptr);
  } catch (const std::invalid_argument&) {
    threw = true;
  }
  EXPECT(threw);
  threw = false;
  try {
    api::grouped_gemm::group_gemm_nvfp4_async(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                                             nullptr, nullptr, 4, 128, 128, 128, 128, 32, true, nullptr);
  } catch (const std::invalid_argument&) {
    threw = true;
  }
  EXPECT(threw);
  return g_failures;
}

static void expect_all(const std::vector<half>& got, float want, const char* what) {
  std::size_t bad = 0;
  for (const half& h : got) bad += (__half2float(h) != want);
  if (bad) {
    std::printf("FAIL %s: %zu of %zu values differ from %g (first %g)\n", what, bad, got.size(), want,
                __half2float(got[0]));
    ++g_failures;
  }
}

static int device_checks() {
  using api::GemmStatus;
  cudaStream_t stream;
  cuda_ok(cudaStreamCreate(&stream), "stream");
  // 1. single GEMM, every value 1.0 (payload 0x22, scale 0x38): C = K; generic, split-K 4, split-K 2
  for (int m : {16, 128, 256, 300}) {
    const int n = 512, k = 1024;
    DeviceBuffer<std::uint8_t> a(api::packed_fp4_bytes(m, k)), b(api::packed_fp4_bytes(n, k));
    DeviceBuffer<std::uint8_t> sfa(api::scale_a_elements(m, n, k)), sfb(api::scale_b_elements(m, n, k));
    DeviceBuffer<half> c(std::size_t(m) * n);
    DeviceBuffer<std::uint8_t> ws(api::nvfp4_gemm_workspace_size_sm120(m, n, k));
    a.fill_bytes(0x22); b.fill_bytes(0x22); sfa.fill_bytes(0x38); sfb.fill_bytes(0x38); c.fill_bytes(0xff);
    EXPECT(api::nvfp4_gemm_sm120(m, n, k, a.ptr, b.ptr, sfa.ptr, sfb.ptr, c.ptr, ws.ptr, ws.count, stream) == GemmStatus::kSuccess);
    cuda_ok(cudaStreamSynchronize(stream), "sync");
    expect_all(c.download(), float(k), "nvfp4_gemm_sm120");
    c.fill_bytes(0xff);
    EXPECT(api::nvfp4_cutlass_gemm_sm120(m, n, k, a.ptr, b.ptr, sfa.ptr, sfb.ptr, c.ptr, nullptr, 0, stream) == GemmStatus::kSuccess);
    cuda_ok(cudaStreamSynchronize(stream), "sync");
    expect_all(c.download(), float(k), "nvfp4_cutlass_gemm_sm120");
    DeviceBuffer<float> cf(std::size_t(m) * n);
    EXPECT(api::nvfp4_cute_gemm_f32_sm120(m, n, k, a.ptr, b.ptr, sfa.ptr, sfb.ptr, cf.ptr, stream) == GemmStatus::kSuccess);
    cuda_ok(cudaStreamSynchronize(stream), "sync");
    for (float v : cf.download()) if (v != float(k)) { std::printf("FAIL f32 gemm value %g\n", v); ++g_failures; break; }
  }
  // 2. grouped GEMM with an empty group and ragged tails; rows outside the groups stay untouched
  {
    const int groups = 4, n = 256, k = 512, m_pad = 256;
    const std::vector<int> seqlens = {129, 0, 1, 127};
    const std::vector<int> cu = {0, 129, 129, 130, 257};
    const int m = 260;
    DeviceBuffer<std::uint8_t> x(api::packed_fp4_bytes(m, k)), w(std::size_t(groups) * api::packed_fp4_bytes(n, k));
    DeviceBuffer<std::uint8_t> xs(std::size_t(groups) * m_pad * api::scale_k_padded(k)), wsf(std::size_t(groups) * api::scale_b_elements(1, n, k));
    DeviceBuffer<half> y(std::size_t(m) * n);
    DeviceBuffer<int> dseq(groups), dcu(groups + 1), tiles(groups), cu_tiles(groups + 1);
    DeviceBuffer<std::uint8_t> tmas(std::size_t(3 * groups + 2) * 128);
    x.fill_bytes(0x22); w.fill_bytes(0x22); xs.fill_bytes(0x38); wsf.fill_bytes(0x38); y.fill_bytes(0);
    dseq.upload(seqlens); dcu.upload(cu);
    api::grouped_gemm::group_gemm_nvfp4_async(y.ptr, x.ptr, w.ptr, dseq.ptr, dcu.ptr, xs.ptr, wsf.ptr, tmas.ptr, tiles.ptr,
                                             cu_tiles.ptr, groups, m, n, k, m_pad, 64, true, stream);
    cuda_ok(cudaStreamSynchronize(stream), "sync");
    const std::vector<half> out = y.download();
    for (int r = 0; r < m; ++r) {
      const float want = r < 257 ? float(k) : 0.0f;
      for (int c0 = 0; c0 < n; c0 += 85)
        if (__half2float(out[std::size_t(r) * n + c0]) != want) { std::printf("FAIL grouped row %d\n", r); ++g_failures; r = m; break; }
    }
    const std::vector<int> t = tiles.download();
    EXPECT(t[0] == 2 && t[1] == 0 && t[2] == 1 && t[3] == 1);
  }
  // 3. routed layer on uniform data: every output is 33792 (1024/6 -> UE4M3 176, 1024/176 -> E2M1 6)
  {
    const int tokens = 4, experts = 2, hidden = 128, inter = 64, topk = 2, total = tokens * topk, m_pad = 128;
    DeviceBuffer<std::uint8_t> x(api::packed_fp4_bytes(tokens, hidden)), xs(128 * api::scale_k_padded(hidden));
    DeviceBuffer<std::uint8_t> gw(std::size_t(experts) * api::packed_fp4_bytes(2 * inter, hidden)), gs(std::size_t(experts) * 128 * api::scale_k_padded(hidden));
    DeviceBuffer<std::uint8_t> dw(std::size_t(experts) * api::packed_fp4_bytes(hidden, inter)), ds(std::size_t(experts) * 128 * api::scale_k_padded(inter));
    x.fill_bytes(0x11); gw.fill_bytes(0x11); dw.fill_bytes(0x11); xs.fill_bytes(0x38); gs.fill_bytes(0x38); ds.fill_bytes(0x38);
    DeviceBuffer<int> ids(total), pos(total), seq(experts), cu(experts + 1), tiles(experts), cu_tiles(experts + 1);
    DeviceBuffer<float> wts(total);
    DeviceBuffer<half> shared(std::size_t(tokens) * hidden), out(std::size_t(tokens) * hidden);
    ids.upload({0, 1, 1, 0, 0, 1, 1, 0});
    wts.upload({0.25f, 0.75f, 0.6f, 0.4f, 0.5f, 0.5f, 0.2f, 0.8f});
    shared.upload(std::vector<half>(std::size_t(tokens) * hidden, __float2half(2.0f)));
    DeviceBuffer<std::uint8_t> gin(api::packed_fp4_bytes(total, hidden)), gin_s(std::size_t(experts) * m_pad * api::scale_k_padded(hidden));
    DeviceBuffer<half> gout(std::size_t(total) * 2 * inter), dout(std::size_t(total) * hidden);
    DeviceBuffer<std::uint8_t> din(api::packed_fp4_bytes(total, inter)), din_s(std::size_t(experts) * m_pad * api::scale_k_padded(inter));
    DeviceBuffer<std::uint8_t> tm1(std::size_t(3 * experts + 2) * 128), tm2(std::size_t(3 * experts + 2) * 128);
    api::fused_moe::fuse_moe_nvfp4_async(out.ptr, x.ptr, xs.ptr, gin.ptr, gin_s.ptr, gout.ptr, gw.ptr, gs.ptr, tm1.ptr, din.ptr,
                                        din_s.ptr, dout.ptr, dw.ptr, ds.ptr, tm2.ptr, ids.ptr, wts.ptr, pos.ptr, seq.ptr, cu.ptr,
                                        tiles.ptr, cu_tiles.ptr, shared.ptr, tokens, hidden, inter, topk, experts, experts, 0,
                                        128, m_pad, stream);
    cuda_ok(cudaStreamSynchronize(stream), "sync");
    expect_all(out.download(), 33792.0f, "fuse_moe_nvfp4_async");
    // the expert-major entry on the rows the routed call gathered: 33792 per expanded row (the
    // routed output adds the shared 2.0, which FP16 rounding absorbs at this magnitude)
    const std::size_t need = api::fused_moe::expert_moe_nvfp4_workspace_size(total, hidden, inter, experts, m_pad);
    DeviceBuffer<std::uint8_t> wsp(need);
    DeviceBuffer<half> rows(std::size_t(total) * hidden);
    api::fused_moe::expert_moe_nvfp4_async(rows.ptr, gin.ptr, gin_s.ptr, gw.ptr, gs.ptr, dw.ptr, ds.ptr, seq.ptr, cu.ptr, wsp.ptr,
                                          need, total, hidden, inter, experts, m_pad, stream);
    cuda_ok(cudaStreamSynchronize(stream), "sync");
    expect_all(rows.download(), 33792.0f, "expert_moe_nvfp4_async");
  }
  cudaStreamDestroy(stream);
  return g_failures;
}

int main(int argc, char** argv) {
  const std::string mode = argc > 1 ? argv[1] : "host";
  int failures = 0;
  try {
    failures = mode == "device" ? (host_checks(), device_checks()) : host_checks();
  } catch (const std::exception& e) {
    std::printf("FAIL exception: %s\n", e.what());
    return 2;
  }
  std::printf(failures ? "FAILED (%d)\n" : "PASS\n", failures);
  return failures ? 1 : 0;
}
