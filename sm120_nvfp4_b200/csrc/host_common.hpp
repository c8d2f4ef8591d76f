// Host-side helpers shared by the launchers: status codes of the C ABI, cached device
// properties, the driver entry point for tensor-map encoding and the device error word.
#pragma once

#include <cstddef>
#include <cstdint>

#include <cuda.h>
#include <cuda_runtime.h>

#include "b200_nvfp4.h"

namespace b200 {

struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0;
  int cc_minor = 0;
  bool ok = false;
};

// Properties of the current device (queried once per device, then cached).
const DeviceInfo& current_device_info();

// True when the current device can run the sm_100a kernels (compute capability 10.x).
bool device_supported(const DeviceInfo& info);

// Encodes a rank-2 tiled tensor map over a row-major byte matrix [rows, row_bytes] with a
// box of [box_rows, box_bytes] and the given swizzle. Returns false on failure.
bool encode_tmap_2d_u8(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                       uint32_t box_rows, uint32_t box_bytes, CUtensorMapSwizzle swizzle);

// Tensor map for TMA stores of an FP16 / FP32 row-major matrix [rows, cols]: box of
// [box_rows, box_cols] elements whose rows are 128 bytes, 128-byte swizzle.
bool encode_tmap_2d_out(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                        bool is_f32, uint32_t box_rows, uint32_t box_cols);

// Rank-3 tiled map over block-scaled scale regions: {128 32-bit words of one 512-byte atom,
// `kt` atoms along K, `atom_rows` 128-row atom rows}, box {128, box_atoms, box_rows}, no swizzle.
// Boxes that reach past an extent are completed with zeros.
bool encode_tmap_sf(CUtensorMap* map, const void* base, uint64_t kt, uint64_t atom_rows, uint32_t box_atoms,
                    uint32_t box_rows);

// Device word written by kernels whose bounded waits time out. One per loaded library.
int* device_error_word();

inline int align_up_int(int x, int a) { return (x + a - 1) / a * a; }
inline int scale_k_padded(int k) { return align_up_int((k + 15) / 16, 4); }

}  // namespace b200
