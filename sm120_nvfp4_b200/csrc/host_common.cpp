#include "host_common.hpp"

#include <atomic>
#include <mutex>

namespace b200 {

namespace {

constexpr int kMaxDevices = 64;
DeviceInfo g_info[kMaxDevices];
std::once_flag g_info_once[kMaxDevices];

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) !=
            cudaSuccess ||
        res != cudaDriverEntryPointSuccess) {
      ptr = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

}  // namespace

const DeviceInfo& current_device_info() {
  static DeviceInfo invalid;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return invalid;
  std::call_once(g_info_once[device], [device] {
    DeviceInfo info;
    info.device = device;
    bool ok = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, device) ==
              cudaSuccess;
    ok = ok && cudaDeviceGetAttribute(&info.cc_major, cudaDevAttrComputeCapabilityMajor, device) ==
                   cudaSuccess;
    ok = ok && cudaDeviceGetAttribute(&info.cc_minor, cudaDevAttrComputeCapabilityMinor, device) ==
                   cudaSuccess;
    info.ok = ok;
    g_info[device] = info;
  });
  return g_info[device];
}

bool device_supported(const DeviceInfo& info) { return info.ok && info.cc_major == 10; }

bool encode_tmap_2d_u8(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                       uint32_t box_rows, uint32_t box_bytes, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {box_bytes, box_rows};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides,
                  box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool encode_tmap_sf(CUtensorMap* map, const void* base, uint64_t kt, uint64_t atom_rows, uint32_t box_atoms,
                    uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr || kt == 0 || atom_rows == 0) return false;
  cuuint64_t dims[3] = {128, kt, atom_rows};
  cuuint64_t strides[2] = {512, kt * 512};
  cuuint32_t box[3] = {128, box_atoms, box_rows};
  cuuint32_t elem_strides[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(base), dims, strides, box,
                  elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Rank-2 tiled map over a row-major matrix of 2- or 4-byte elements (store side: no L2
// promotion).
bool encode_tmap_2d_out(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                        bool is_f32, uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  const uint64_t elem = is_f32 ? 4 : 2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * elem};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = fn(map, is_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace b200
