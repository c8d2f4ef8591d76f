// NVFP4 GEMM on operands that live in host memory: C_host = A_host x B_host^T, with the copies
// in both directions overlapped with the arithmetic.
//
// A caller that holds its operands on the host pays for three things in sequence when it uses the
// device-pointer entry points: host -> device copies, the kernel, the device -> host copy of C.
// For the shapes this library is built for the kernel is the smallest of the three (8192^3: 0.2 ms
// of arithmetic between 1.4 ms and 2.6 ms of copies), and the link is full duplex. This entry
// point therefore cuts A into row chunks and B into row chunks (= column blocks of C), uploads
// them alternately, launches the GEMM of a block of C as soon as its A chunk and its B chunk
// have landed, and sends the block home while later chunks are still arriving: after the first
// two chunks the device -> host direction is busy until the end.
//
// The library allocates no device memory: the caller passes device scratch for the operands and
// for C. Streams and events are host-side objects, created once per device on first use.
// Host buffers should be page-locked, otherwise the copies are staged by the driver and overlap
// less. On return all work is enqueued and `stream` has been made to wait for the last copy, so
// synchronising `stream` (or recording an event on it) is enough to read C_host.
#include <cstddef>
#include <cstdint>
#include <mutex>
#include <vector>

#include <cuda_runtime.h>

#include "b200_nvfp4.h"

namespace b200 {
namespace {

constexpr int kMaxDevices = 64;
constexpr int kMaxChunks = 64;                       // per operand
constexpr int kMaxBlocks = 1024;                     // blocks of C per call

struct HostGemmResources {
  cudaStream_t up = nullptr, down = nullptr;         // copy streams, one per direction
  std::vector<cudaEvent_t> events;                   // chunk landed / block computed / call begin / call end
  bool ok = false;
};

HostGemmResources* resources_for_current_device() {
  static HostGemmResources table[kMaxDevices];
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return nullptr;
  HostGemmResources& r = table[device];
  if (!r.ok) {
    if (cudaStreamCreateWithFlags(&r.up, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaStreamCreateWithFlags(&r.down, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    r.events.resize(2 * kMaxChunks + kMaxBlocks + 2);
    for (cudaEvent_t& e : r.events)
      if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    r.ok = true;
  }
  return &r;
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// bytes of the scale region of `rows` rows (a multiple of 128 but for the last chunk) with k columns
inline size_t scale_bytes(int rows, int k) {
  return align_up(static_cast<size_t>(rows), 128) * align_up((static_cast<size_t>(k) + 15) / 16, 4);
}

}  // namespace
}  // namespace b200

extern "C" {

int b200_nvfp4_gemm_host(int m, int n, int k, const void* a_host, const void* b_host,
                         const void* sfa_host, const void* sfb_host, void* c_host_f16, void* a_dev,
                         void* b_dev, void* sfa_dev, void* sfb_dev, void* c_dev, int block_rows,
                         int block_cols, b200_stream_t stream_handle) {
  using namespace b200;
  if (m <= 0 || n <= 0 || k <= 0 || (k % 32) != 0 || (n % 8) != 0) return B200_NVFP4_INVALID_ARGUMENT;
  if (!a_host || !b_host || !sfa_host || !sfb_host || !c_host_f16 || !a_dev || !b_dev || !sfa_dev ||
      !sfb_dev || !c_dev)
    return B200_NVFP4_INVALID_ARGUMENT;
  if (block_rows == 0) block_rows = 2048;
  if (block_cols == 0) block_cols = 2048;
  // chunks start on scale-atom boundaries (128 rows), so a chunk's scales are one contiguous range
  if (block_rows < 128 || block_cols < 128 || (block_rows % 128) != 0 || (block_cols % 128) != 0)
    return B200_NVFP4_INVALID_ARGUMENT;
  const int na = (m + block_rows - 1) / block_rows, nb = (n + block_cols - 1) / block_cols;
  if (na > kMaxChunks || nb > kMaxChunks || na * nb > kMaxBlocks) return B200_NVFP4_INVALID_ARGUMENT;

  static std::mutex mu;   // the per-device streams and events serve one call at a time
  std::lock_guard<std::mutex> lock(mu);
  HostGemmResources* res = resources_for_current_device();
  if (res == nullptr) return B200_NVFP4_CUDA_ERROR;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  cudaEvent_t* ev_a = res->events.data();
  cudaEvent_t* ev_b = ev_a + kMaxChunks;
  cudaEvent_t* ev_c = ev_b + kMaxChunks;
  cudaEvent_t ev_begin = ev_c[kMaxBlocks], ev_end = ev_c[kMaxBlocks + 1];

  bool cuda_ok = true;
  auto check = [&](cudaError_t e) { cuda_ok = cuda_ok && e == cudaSuccess; };
  // the scratch may still be read or written by work queued on `stream` before this call
  check(cudaEventRecord(ev_begin, stream));
  check(cudaStreamWaitEvent(res->up, ev_begin, 0));
  check(cudaStreamWaitEvent(res->down, ev_begin, 0));

  const size_t row_bytes = static_cast<size_t>(k) / 2;
  const size_t skp = align_up((static_cast<size_t>(k) + 15) / 16, 4);   // scale bytes per row
  auto rows_of = [&](int i) { return i + 1 < na ? block_rows : m - i * block_rows; };
  auto cols_of = [&](int j) { return j + 1 < nb ? block_cols : n - j * block_cols; };
  auto upload = [&](const void* payload, const void* scales, void* payload_dev, void* scales_dev, int row0,
                    int rows, cudaEvent_t landed) {
    const size_t off = static_cast<size_t>(row0) * row_bytes, soff = static_cast<size_t>(row0) * skp;
    check(cudaMemcpyAsync(static_cast<uint8_t*>(payload_dev) + off, static_cast<const uint8_t*>(payload) + off,
                          static_cast<size_t>(rows) * row_bytes, cudaMemcpyHostToDevice, res->up));
    check(cudaMemcpyAsync(static_cast<uint8_t*>(scales_dev) + soff, static_cast<const uint8_t*>(scales) + soff,
                          scale_bytes(rows, k), cudaMemcpyHostToDevice, res->up));
    check(cudaEventRecord(landed, res->up));
  };
  int status = B200_NVFP4_SUCCESS;
  // Block (i, j) of C is kept dense ([rows_i, cols_j]) in the scratch, band after band, and goes
  // home with a pitched copy.
  auto block = [&](int i, int j) {
    if (status != B200_NVFP4_SUCCESS) return;
    const int rows = rows_of(i), cols = cols_of(j);
    const size_t row0 = static_cast<size_t>(i) * block_rows, col0 = static_cast<size_t>(j) * block_cols;
    uint8_t* c_blk = static_cast<uint8_t*>(c_dev) + (row0 * n + static_cast<size_t>(rows) * col0) * 2;
    status = b200_nvfp4_gemm(1, rows, cols, k, static_cast<const uint8_t*>(a_dev) + row0 * row_bytes,
                             static_cast<const uint8_t*>(b_dev) + col0 * row_bytes,
                             static_cast<const uint8_t*>(sfa_dev) + row0 * skp,
                             static_cast<const uint8_t*>(sfb_dev) + col0 * skp, c_blk, 0, stream);
    if (status != B200_NVFP4_SUCCESS) return;
    cudaEvent_t done = ev_c[i * nb + j];
    check(cudaEventRecord(done, stream));
    check(cudaStreamWaitEvent(res->down, done, 0));
    check(cudaMemcpy2DAsync(static_cast<uint8_t*>(c_host_f16) + (row0 * n + col0) * 2, static_cast<size_t>(n) * 2,
                            c_blk, static_cast<size_t>(cols) * 2, static_cast<size_t>(cols) * 2,
                            static_cast<size_t>(rows), cudaMemcpyDeviceToHost, res->down));
  };
  // Upload order A0, B0, A1, B1, ...: every chunk that lands completes a row or a column of the
  // grid of blocks that can run, so the number of runnable blocks grows with the square of the
  // bytes uploaded and the way home does not starve.
  int loaded_a = 0, loaded_b = 0;
  while (loaded_a < na || loaded_b < nb) {
    if (loaded_a < na && (loaded_a <= loaded_b || loaded_b == nb)) {
      const int i = loaded_a++;
      upload(a_host, sfa_host, a_dev, sfa_dev, i * block_rows, rows_of(i), ev_a[i]);
      check(cudaStreamWaitEvent(stream, ev_a[i], 0));
      for (int j = 0; j < loaded_b; ++j) block(i, j);
    } else {
      const int j = loaded_b++;
      upload(b_host, sfb_host, b_dev, sfb_dev, j * block_cols, cols_of(j), ev_b[j]);
      check(cudaStreamWaitEvent(stream, ev_b[j], 0));
      for (int i = 0; i < loaded_a; ++i) block(i, j);
    }
  }
  check(cudaEventRecord(ev_end, res->down));
  check(cudaStreamWaitEvent(stream, ev_end, 0));
  if (status != B200_NVFP4_SUCCESS) return status;
  return cuda_ok ? B200_NVFP4_SUCCESS : B200_NVFP4_CUDA_ERROR;
}

}  // extern "C"
