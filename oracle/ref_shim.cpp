// Thin C wrapper around code the reference itself compiles and calls, so the
// oracle's restatement can be checked against the real thing on the CPU.
//
// TEST INFRASTRUCTURE ONLY. Built by oracle/build.py (only where the reference
// checkout is present) into oracle/_ref/libref_shim.so. It includes, where
// they lie, the reference's own header src/fused_moe/scale_layout.cuh (the
// sfa_offset / sfb_offset helpers, lines 33-54) and the third-party pieces the
// reference's quantiser calls: cutlass::float_ue4m3_t and cutlass::float_e2m1_t
// (src/fused_moe/activation.cu:61-72, tests/cpp/test_gemm.cu:37-51; CUTLASS is
// un-vendored, "4.2+", cmake/Dependencies.cmake:3-17 - the headers used here
// are the CUTLASS copy bundled with the flashinfer Python package) and the
// CUDA toolkit's host implementation of the E2M1 pack in <cuda_fp4.h>
// (activation.cu:81). No reference source is copied.
#include <cstdint>

#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "cutlass/float8.h"
#include "cutlass/float_subbyte.h"
#include "fused_moe/scale_layout.cuh"

extern "C" {

int64_t ref_sfa_offset(int row, int k_block, int m_pad, int logical_k) {
  return sm120_nvfp4::fused_moe::sfa_offset(row, k_block, m_pad, logical_k);
}

int64_t ref_sfb_offset(int column, int k_block, int logical_n, int logical_k) {
  return sm120_nvfp4::fused_moe::sfb_offset(column, k_block, logical_n, logical_k);
}

int64_t ref_sfa_group_elements(int m_pad, int k) {
  return sm120_nvfp4::fused_moe::sfa_group_elements(m_pad, k);
}

// CUTLASS host conversion (software path; the device path is the PTX cvt).
uint8_t ref_cutlass_ue4m3_encode(float x) { return cutlass::float_ue4m3_t(x).raw(); }

float ref_cutlass_ue4m3_decode(uint8_t b) {
  return static_cast<float>(cutlass::float_ue4m3_t::bitcast(b));
}

uint8_t ref_cutlass_e2m1_encode(float x) {
  return static_cast<uint8_t>(cutlass::float_e2m1_t(x).raw() & 0x0f);
}

float ref_cutlass_e2m1_decode(uint8_t nibble) {
  return static_cast<float>(cutlass::float_e2m1_t::bitcast(static_cast<uint8_t>(nibble & 0x0f)));
}

// CUDA toolkit host emulation of cvt.rn.satfinite.{e2m1x2,e4m3x2}.f32.
uint8_t ref_cuda_e2m1_encode(float x) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp4(x, __NV_E2M1, cudaRoundNearest) & 0x0f);
}

uint8_t ref_cuda_e4m3_encode(float x) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}

}  // extern "C"
