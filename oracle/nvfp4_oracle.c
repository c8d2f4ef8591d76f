/*
 * CPU oracle for the NVFP4 GEMM -> grouped GEMM -> fused-MoE path.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the shipped library links or calls this
 * file; it is the checker used by tests/, by the smoke entry and by the CPU
 * baseline leg of bench.py.
 *
 * It restates, in plain C, the semantics of the reference implementation
 * (xinyang-zhou/sm120_nvfp4_ops). Each function names the reference file:line
 * it follows. Parity pins: the reference's own known-answer tests
 * (all-ones -> K, the 0x11 MoE case -> 33792 / 8448, dyadic random payloads,
 * the scale-offset formula of tests/python/test_fused_moe.py:160-168) and the
 * CUTLASS / CUDA-toolkit host conversions the reference calls
 * (cutlass::float_ue4m3_t, cutlass::float_e2m1_t, __nv_cvt_float_to_fp4),
 * compiled from their own headers by oracle/build.py into oracle/_ref/.
 * The accumulation order inside the reference's tensor-core MMA is not pinned
 * by any reference test ("parity unpinned" for that detail only): every
 * reference test uses exactly representable sums, so the GEMM oracle computes
 * the exact sum (double accumulation of exact block partials) and the GPU is
 * compared under the stated tolerance.
 *
 * Build: gcc -O3 -march=native -fopenmp -ffp-contract=off -shared -fPIC
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* Number formats                                                            */
/* ------------------------------------------------------------------------- */

/* E2M1 code points, sign in bit 3 (tests/python/test_gemm.py:21-22). */
static const float kE2M1[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f,
                                -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};
/* Twice the E2M1 value, as small integers, so block dot products are exact. */
static const int8_t kE2M1x2[16] = {0, 1, 2, 3, 4, 6, 8, 12,
                                   0, -1, -2, -3, -4, -6, -8, -12};

ORACLE_API float oracle_e2m1_decode(uint8_t nibble) { return kE2M1[nibble & 15]; }

/* Round-to-nearest-even onto the E2M1 grid, saturating at +-6; the reference
 * packs pairs with __nv_fp4x2_e2m1(float2) (src/fused_moe/activation.cu:77-83),
 * i.e. cvt.rn.satfinite.e2m1x2.f32. Ties go to the even CODE. NaN -> +6. */
ORACLE_API uint8_t oracle_e2m1_encode(float x) {
  uint8_t sign = signbit(x) ? 8 : 0;
  float a = fabsf(x);
  uint8_t code;
  if (isnan(x)) return 7;
  if (a <= 0.25f) code = 0;
  else if (a < 0.75f) code = 1;
  else if (a <= 1.25f) code = 2;
  else if (a < 1.75f) code = 3;
  else if (a <= 2.5f) code = 4;
  else if (a < 3.5f) code = 5;
  else if (a <= 5.0f) code = 6;
  else code = 7;
  return (uint8_t)(sign | code);
}

/* UE4M3 = the non-negative half of E4M3 (bias 7, 0x38 = 1.0, 0x7e = 448,
 * 0x7f = NaN); docs/API.md:11, include/sm120_nvfp4/gemm.hpp:13-17. */
ORACLE_API float oracle_ue4m3_decode(uint8_t b) {
  int e = (b >> 3) & 15, m = b & 7;
  float v;
  if ((b & 0x7f) == 0x7f) return NAN;
  if (e == 0) v = ldexpf((float)m, -9);
  else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
  return (b & 0x80) ? -v : v;
}

/* cutlass::float_ue4m3_t(float) as the reference's device code runs it:
 * cvt.rn.satfinite.e4m3x2.f32 (round to nearest even, finite saturation to
 * 448, NaN -> 0x7f). src/fused_moe/activation.cu:61-72. */
ORACLE_API uint8_t oracle_ue4m3_encode(float x) {
  uint32_t bits;
  uint8_t sign;
  float a;
  if (isnan(x)) return 0x7f;
  sign = signbit(x) ? 0x80 : 0;
  a = fabsf(x);
  if (a >= 448.0f) return (uint8_t)(sign | 0x7e);
  if (a < 0.015625f) { /* below the smallest normal 2^-6: multiples of 2^-9 */
    float q = rintf(a * 512.0f); /* exact scaling, ties to even */
    return (uint8_t)(sign | (uint8_t)q); /* q==8 is the smallest normal 0x08 */
  }
  memcpy(&bits, &a, 4);
  {
    uint32_t lsb = (bits >> 20) & 1u;
    uint32_t r = bits + 0x7ffffu + lsb; /* RNE to 3 mantissa bits */
    int e = (int)((r >> 23) & 0xff) - 127 + 7;
    uint32_t m = (r >> 20) & 7u;
    uint32_t code = ((uint32_t)e << 3) | m;
    if (code > 0x7e) code = 0x7e;
    return (uint8_t)(sign | code);
  }
}

/* IEEE binary16 <-> binary32, round to nearest even (__float2half_rn). */
ORACLE_API uint16_t oracle_f32_to_f16(float f) {
  uint32_t x;
  uint32_t sign, mant;
  int exp;
  memcpy(&x, &f, 4);
  sign = (x >> 16) & 0x8000u;
  exp = (int)((x >> 23) & 0xff);
  mant = x & 0x7fffffu;
  if (exp == 0xff) return (uint16_t)(sign | 0x7c00u | (mant ? 0x200u : 0));
  exp = exp - 127 + 15;
  if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
  if (exp <= 0) {
    uint32_t shift, halfbit, rem, res;
    if (exp < -10) return (uint16_t)sign;
    mant |= 0x800000u;
    shift = (uint32_t)(14 - exp);
    res = mant >> shift;
    halfbit = 1u << (shift - 1);
    rem = mant & ((1u << shift) - 1);
    if (rem > halfbit || (rem == halfbit && (res & 1))) res++;
    return (uint16_t)(sign | res);
  }
  {
    uint32_t res = ((uint32_t)exp << 10) | (mant >> 13);
    uint32_t rem = mant & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (res & 1))) res++;
    return (uint16_t)(sign | res);
  }
}

ORACLE_API float oracle_f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  int exp = (h >> 10) & 31;
  uint32_t mant = h & 0x3ffu;
  uint32_t out;
  float f;
  if (exp == 0) {
    if (mant == 0) out = sign;
    else {
      int e = -1;
      do { mant <<= 1; e++; } while (!(mant & 0x400u));
      out = sign | ((uint32_t)(127 - 15 - e) << 23) | ((mant & 0x3ffu) << 13);
    }
  } else if (exp == 31) out = sign | 0x7f800000u | (mant << 13);
  else out = sign | ((uint32_t)(exp - 15 + 127) << 23) | (mant << 13);
  memcpy(&f, &out, 4);
  return f;
}

ORACLE_API float oracle_bf16_to_f32(uint16_t h) {
  uint32_t out = (uint32_t)h << 16;
  float f;
  memcpy(&f, &out, 4);
  return f;
}

ORACLE_API uint16_t oracle_f32_to_bf16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40);
  x += 0x7fffu + ((x >> 16) & 1u);
  return (uint16_t)(x >> 16);
}

/* ------------------------------------------------------------------------- */
/* Scale-factor layout                                                       */
/* ------------------------------------------------------------------------- */

/* include/sm120_nvfp4/gemm.hpp:39-42 */
ORACLE_API int oracle_scale_k_padded(int k) { return (((k + 15) / 16) + 3) / 4 * 4; }

/* Byte offset of the scale of (row, k_block) inside one physical region of the
 * block-scaled layout the reference obtains from
 * Sm1xxBlockScaledConfig<16>::tile_atom_to_shape_SFA
 * (src/fused_moe/scale_layout.cuh:33-41): 512-byte atoms of 128 rows x 4
 * k-blocks, atoms K-major inside a 128-row tile. The closed form is the one
 * tests/python/test_fused_moe.py:160-168 writes out for its first atom row. */
ORACLE_API int64_t oracle_sf_offset(int row, int k_block, int k) {
  int64_t kt = oracle_scale_k_padded(k) / 4;
  return ((int64_t)(row / 128) * kt + k_block / 4) * 512 + (row % 32) * 16 +
         ((row % 128) / 32) * 4 + (k_block % 4);
}

/* ------------------------------------------------------------------------- */
/* Quantiser                                                                 */
/* ------------------------------------------------------------------------- */

/* One 16-element block: src/fused_moe/activation.cu:58-84 (and :141-161).
 * amax/6 -> UE4M3 (RNE, saturating); a non-zero block whose scale rounds to
 * zero gets raw code 1; payload = value / decoded scale -> E2M1 RNE. A zero
 * block has scale byte 0 and payload 0. */
static uint8_t quantize_block16(const float *v, uint8_t *payload8) {
  float amax = 0.0f;
  uint8_t code = 0;
  float decoded = 1.0f;
  int i;
  for (i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  if (amax > 0.0f) {
    code = oracle_ue4m3_encode(amax / 6.0f);
    decoded = oracle_ue4m3_decode(code);
    if (!(decoded > 0.0f)) {
      code = 1;
      decoded = oracle_ue4m3_decode(code);
    }
  }
  for (i = 0; i < 8; ++i) {
    uint8_t lo = oracle_e2m1_encode(v[2 * i] / decoded);
    uint8_t hi = oracle_e2m1_encode(v[2 * i + 1] / decoded);
    payload8[i] = (uint8_t)(lo | (hi << 4)); /* low nibble = even k */
  }
  return code;
}

/* Row-wise NVFP4 quantisation of an FP32 matrix [rows, k] into packed payload
 * [rows, k/2] and one scale region of align128(rows) * scale_k_padded(k) bytes
 * (zero-filled first). Used to make GEMM inputs from seeded N(0,1) data with
 * the same rules as the reference's quantiser. */
ORACLE_API void oracle_quantize_rows_f32(const float *x, int rows, int k,
                                         uint8_t *packed, uint8_t *scales) {
  int skp = oracle_scale_k_padded(k);
  int64_t region = (int64_t)((rows + 127) / 128 * 128) * skp;
  int r;
  memset(scales, 0, (size_t)region);
#pragma omp parallel for schedule(static)
  for (r = 0; r < rows; ++r) {
    int kb;
    for (kb = 0; kb < k / 16; ++kb) {
      uint8_t code = quantize_block16(x + (int64_t)r * k + kb * 16,
                                      packed + (int64_t)r * (k / 2) + kb * 8);
      scales[oracle_sf_offset(r, kb, k)] = code;
    }
  }
}

/* ------------------------------------------------------------------------- */
/* GEMM                                                                      */
/* ------------------------------------------------------------------------- */

static void unpack_row_x2(const uint8_t *packed, int k, int8_t *out) {
  int i;
  for (i = 0; i < k / 2; ++i) {
    out[2 * i] = kE2M1x2[packed[i] & 15];
    out[2 * i + 1] = kE2M1x2[packed[i] >> 4];
  }
}

/* C[r, c] = sum_k (A[r,k] * SFA[r,k/16]) * (B[c,k] * SFB[c,k/16]) for the
 * listed rows and columns; tests/cpp/test_gemm.cu:216-227 with per-block
 * scales (include/sm120_nvfp4/gemm.hpp:133-142). Each 16-element block
 * partial is exact in FP32 (an integer dot product of doubled codes times the
 * product of two 4-bit-mantissa scales); blocks are summed in double and the
 * result is rounded once to FP32. alpha multiplies in FP32 before the store.
 * row_idx / col_idx may be NULL (identity). out is [n_rows, n_cols] FP32. */
ORACLE_API void oracle_gemm_sampled(int m, int n, int k, const uint8_t *a,
                                    const uint8_t *b, const uint8_t *sfa,
                                    const uint8_t *sfb, const int *row_idx,
                                    int n_rows, const int *col_idx, int n_cols,
                                    float alpha, float *out) {
  int kb_count = k / 16;
  int8_t *ua = (int8_t *)malloc((size_t)n_rows * k);
  float *sa = (float *)malloc((size_t)n_rows * kb_count * sizeof(float));
  int i;
  (void)m;
  (void)n;
  for (i = 0; i < n_rows; ++i) {
    int r = row_idx ? row_idx[i] : i, kb;
    unpack_row_x2(a + (int64_t)r * (k / 2), k, ua + (int64_t)i * k);
    for (kb = 0; kb < kb_count; ++kb)
      sa[(int64_t)i * kb_count + kb] =
          oracle_ue4m3_decode(sfa[oracle_sf_offset(r, kb, k)]);
  }
#pragma omp parallel
  {
    int8_t *ub = (int8_t *)malloc((size_t)k);
    float *sb = (float *)malloc((size_t)kb_count * sizeof(float));
    int j;
#pragma omp for schedule(dynamic, 4)
    for (j = 0; j < n_cols; ++j) {
      int c = col_idx ? col_idx[j] : j, kb, ii;
      unpack_row_x2(b + (int64_t)c * (k / 2), k, ub);
      for (kb = 0; kb < kb_count; ++kb)
        sb[kb] = oracle_ue4m3_decode(sfb[oracle_sf_offset(c, kb, k)]);
      for (ii = 0; ii < n_rows; ++ii) {
        const int8_t *pa = ua + (int64_t)ii * k;
        const float *psa = sa + (int64_t)ii * kb_count;
        double acc = 0.0;
        for (kb = 0; kb < kb_count; ++kb) {
          int dot = 0, t;
          for (t = 0; t < 16; ++t) dot += (int)pa[kb * 16 + t] * (int)ub[kb * 16 + t];
          /* doubled codes on both sides -> divide by 4; exact in FP32 */
          acc += (double)((float)dot * 0.25f * (psa[kb] * sb[kb]));
        }
        out[(int64_t)ii * n_cols + j] = (float)acc * alpha;
      }
    }
    free(ub);
    free(sb);
  }
  free(ua);
  free(sa);
}

/* Full GEMM; writes FP32 and/or FP16 (RNE, static_cast<half_t> in
 * src/gemm/cute_gemm.cu:282-289). Either output may be NULL. */
ORACLE_API void oracle_gemm(int m, int n, int k, const uint8_t *a, const uint8_t *b,
                            const uint8_t *sfa, const uint8_t *sfb, float alpha,
                            float *c_f32, uint16_t *c_f16) {
  float *tmp = c_f32 ? c_f32 : (float *)malloc((size_t)m * n * sizeof(float));
  int64_t i;
  oracle_gemm_sampled(m, n, k, a, b, sfa, sfb, NULL, m, NULL, n, alpha, tmp);
  if (c_f16)
    for (i = 0; i < (int64_t)m * n; ++i) c_f16[i] = oracle_f32_to_f16(tmp[i]);
  if (!c_f32) free(tmp);
}

/* Grouped GEMM, include/sm120_nvfp4/grouped_gemm.hpp:9-21 and the epilogue of
 * src/grouped_gemm/kernels.cuh:436-446: rows of expert e are
 * [cu_seqlens[e], cu_seqlens[e]+seqlens[e]); its activation scales live in an
 * own region of m_scale_pad * skp bytes indexed by the row inside the expert;
 * weights [G, n, k/2] and weight scales [G, align128(n) * skp]. Rows outside
 * every expert are left untouched. group_alpha may be NULL (the reference has
 * no such argument; NULL reproduces it). */
ORACLE_API void oracle_grouped_gemm(uint16_t *y, const uint8_t *x, const uint8_t *w,
                                    const int *seqlens, const int *cu_seqlens,
                                    const uint8_t *x_scale, const uint8_t *w_scale,
                                    int num_group, int n, int k, int m_scale_pad,
                                    const float *group_alpha) {
  int skp = oracle_scale_k_padded(k);
  int64_t sfa_stride = (int64_t)m_scale_pad * skp;
  int64_t sfb_stride = (int64_t)((n + 127) / 128 * 128) * skp;
  int g;
  for (g = 0; g < num_group; ++g) {
    int rows = seqlens[g];
    if (rows <= 0) continue;
    oracle_gemm(rows, n, k, x + (int64_t)cu_seqlens[g] * (k / 2),
                w + (int64_t)g * n * (k / 2), x_scale + g * sfa_stride,
                w_scale + g * sfb_stride, group_alpha ? group_alpha[g] : 1.0f,
                NULL, y + (int64_t)cu_seqlens[g] * n);
  }
}

/* Split-K reduction: src/gemm/specialized/m128_gemm.cu:367-382. */
ORACLE_API void oracle_splitk_reduce(const float *partial, int splits, int64_t numel,
                                     uint16_t *out) {
  int64_t i;
  for (i = 0; i < numel; ++i) {
    float s = 0.0f;
    int p;
    for (p = 0; p < splits; ++p) s += partial[(int64_t)p * numel + i];
    out[i] = oracle_f32_to_f16(s);
  }
}

/* ------------------------------------------------------------------------- */
/* MoE glue                                                                  */
/* ------------------------------------------------------------------------- */

/* src/fused_moe/count_and_gather.cu:12-92,96-143. Local experts are
 * [rank_ep*E, rank_ep*E+E). The reference assigns slots inside an expert with
 * atomics (order unspecified, :59-64); the canonical order used here - and by
 * the CUDA path - is ascending flat assignment index t*k+r, which is one of
 * the reference's possible outcomes. Scale output is zero-filled first
 * (:112-116). seqlens ends as the per-expert count (reset then re-counted). */
ORACLE_API void oracle_count_and_gather(uint8_t *grouped_input, uint8_t *grouped_scale,
                                        const uint8_t *input, const uint8_t *input_scale,
                                        const int *topk_ids, int *topk_pos, int *seqlens,
                                        int *cu_seqlens, int num_tokens, int hidden,
                                        int num_topk, int num_expert_local, int rank_ep,
                                        int input_scale_m_pad, int grouped_scale_m_pad) {
  int total = num_tokens * num_topk;
  int start = rank_ep * num_expert_local, end = start + num_expert_local;
  int skp = oracle_scale_k_padded(hidden);
  int64_t group_stride = (int64_t)grouped_scale_m_pad * skp;
  int *fill = (int *)calloc((size_t)num_expert_local, sizeof(int));
  int a, e;
  (void)input_scale_m_pad;
  memset(seqlens, 0, (size_t)num_expert_local * sizeof(int));
  memset(grouped_scale, 0, (size_t)(num_expert_local * group_stride));
  for (a = 0; a < total; ++a) {
    topk_pos[a] = -1;
    if (topk_ids[a] >= start && topk_ids[a] < end) seqlens[topk_ids[a] - start]++;
  }
  cu_seqlens[0] = 0;
  for (e = 0; e < num_expert_local; ++e) cu_seqlens[e + 1] = cu_seqlens[e] + seqlens[e];
  for (a = 0; a < total; ++a) {
    int eg = topk_ids[a], position, row, token, kb;
    if (eg < start || eg >= end) continue;
    e = eg - start;
    position = fill[e]++;
    row = cu_seqlens[e] + position;
    token = a / num_topk;
    memcpy(grouped_input + (int64_t)row * (hidden / 2),
           input + (int64_t)token * (hidden / 2), (size_t)(hidden / 2));
    for (kb = 0; kb < (hidden + 15) / 16; ++kb)
      grouped_scale[e * group_stride + oracle_sf_offset(position, kb, hidden)] =
          input_scale[oracle_sf_offset(token, kb, hidden)];
    topk_pos[a] = row;
  }
  free(fill);
}

/* exp(x) in FP32 from explicit fused-multiply-adds, so the same operation
 * sequence gives the same bits on the host and on the GPU (the reference calls
 * CUDA's expf, src/fused_moe/activation.cu:17-19, whose bits no CPU libm
 * reproduces). Cody-Waite reduction by ln2, degree-7 polynomial, scaling by
 * two exact powers of two. Error < 2 ulp against a correctly rounded exp. */
ORACLE_API float oracle_expf(float x) {
  float t, n, r, p, s1, s2;
  int ni, h1, h2;
  uint32_t b1, b2;
  if (x > 88.75f) return INFINITY;
  if (x < -104.0f) return 0.0f;
  t = x * 1.44269504088896341f;
  n = rintf(t);
  r = fmaf(n, -0.693145751953125f, x);
  r = fmaf(n, -1.428606765330187045e-06f, r);
  p = 1.0f / 5040.0f;
  p = fmaf(p, r, 1.0f / 720.0f);
  p = fmaf(p, r, 1.0f / 120.0f);
  p = fmaf(p, r, 1.0f / 24.0f);
  p = fmaf(p, r, 1.0f / 6.0f);
  p = fmaf(p, r, 0.5f);
  p = fmaf(p, r, 1.0f);
  p = fmaf(p, r, 1.0f);
  ni = (int)n;
  h1 = ni / 2;
  h2 = ni - h1;
  b1 = (uint32_t)(h1 + 127) << 23;
  b2 = (uint32_t)(h2 + 127) << 23;
  memcpy(&s1, &b1, 4);
  memcpy(&s2, &b2, 4);
  return (p * s1) * s2;
}

/* src/fused_moe/activation.cu:17-19 */
ORACLE_API float oracle_silu(float x) { return x / (1.0f + oracle_expf(-x)); }

/* src/fused_moe/activation.cu:21-90,170-195: gate_up FP16 [rows, 2I] ->
 * payload [rows, I/2] + per-expert scale regions (zero-filled first). */
ORACLE_API void oracle_act_mul_and_quant(uint8_t *output, uint8_t *output_scale,
                                         const uint16_t *gate_up, const int *seqlens,
                                         const int *cu_seqlens, int num_expert_local,
                                         int m_scale_pad, int inter) {
  int skp = oracle_scale_k_padded(inter);
  int64_t group_stride = (int64_t)m_scale_pad * skp;
  int e;
  memset(output_scale, 0, (size_t)(num_expert_local * group_stride));
  for (e = 0; e < num_expert_local; ++e) {
    int row;
#pragma omp parallel for schedule(static)
    for (row = 0; row < seqlens[e]; ++row) {
      int64_t grow = (int64_t)cu_seqlens[e] + row;
      const uint16_t *gate = gate_up + grow * inter * 2;
      const uint16_t *up = gate + inter;
      int kb, i;
      for (kb = 0; kb < inter / 16; ++kb) {
        float v[16];
        for (i = 0; i < 16; ++i)
          v[i] = oracle_silu(oracle_f16_to_f32(gate[kb * 16 + i])) *
                 oracle_f16_to_f32(up[kb * 16 + i]);
        output_scale[e * group_stride + oracle_sf_offset(row, kb, inter)] =
            quantize_block16(v, output + grow * (inter / 2) + kb * 8);
      }
    }
  }
}

/* src/fused_moe/activation.cu:105-166,197-232 */
ORACLE_API void oracle_quantize_expert(uint8_t *output, uint8_t *output_scale,
                                       const uint16_t *input, const int *seqlens,
                                       const int *cu_seqlens, int num_expert_local,
                                       int hidden, int m_scale_pad, int input_is_bf16) {
  int skp = oracle_scale_k_padded(hidden);
  int64_t group_stride = (int64_t)m_scale_pad * skp;
  int e;
  memset(output_scale, 0, (size_t)(num_expert_local * group_stride));
  for (e = 0; e < num_expert_local; ++e) {
    int row;
#pragma omp parallel for schedule(static)
    for (row = 0; row < seqlens[e]; ++row) {
      int64_t grow = (int64_t)cu_seqlens[e] + row;
      const uint16_t *in = input + grow * hidden;
      int kb, i;
      for (kb = 0; kb < hidden / 16; ++kb) {
        float v[16];
        for (i = 0; i < 16; ++i)
          v[i] = input_is_bf16 ? oracle_bf16_to_f32(in[kb * 16 + i])
                               : oracle_f16_to_f32(in[kb * 16 + i]);
        output_scale[e * group_stride + oracle_sf_offset(row, kb, hidden)] =
            quantize_block16(v, output + grow * (hidden / 2) + kb * 8);
      }
    }
  }
}

/* src/fused_moe/reduce.cu:12-35. FP32 accumulation in route order starting
 * from the shared-expert row; "value += x * w" in the reference's device code
 * is contracted by nvcc's default -fmad=true, hence fmaf. */
ORACLE_API void oracle_reduce(uint16_t *output, const uint16_t *down_output,
                              const int *topk_pos, const float *topk_scale,
                              const uint16_t *shared_output, int num_tokens, int hidden,
                              int num_topk) {
  int t;
#pragma omp parallel for schedule(static)
  for (t = 0; t < num_tokens; ++t) {
    int c, r;
    for (c = 0; c < hidden; ++c) {
      float v = shared_output ? oracle_f16_to_f32(shared_output[(int64_t)t * hidden + c]) : 0.0f;
      for (r = 0; r < num_topk; ++r) {
        int row = topk_pos[t * num_topk + r];
        if (row >= 0)
          v = fmaf(oracle_f16_to_f32(down_output[(int64_t)row * hidden + c]),
                   topk_scale[t * num_topk + r], v);
      }
      output[(int64_t)t * hidden + c] = oracle_f32_to_f16(v);
    }
  }
}

/* src/fused_moe/fused_moe.cu:97-157: gate/up grouped GEMM -> SiLU*up + quant
 * -> down grouped GEMM on already expert-major rows. Output FP16 [rows, H]. */
ORACLE_API void oracle_expert_moe(uint16_t *output, const uint8_t *input,
                                  const uint8_t *input_scale, const uint8_t *gate_up_w,
                                  const uint8_t *gate_up_ws, const uint8_t *down_w,
                                  const uint8_t *down_ws, const int *seqlens,
                                  const int *cu_seqlens, int total_rows, int hidden,
                                  int inter, int num_expert_local, int m_scale_pad) {
  int skp_i = oracle_scale_k_padded(inter);
  uint16_t *gate_up = (uint16_t *)calloc((size_t)total_rows * inter * 2, 2);
  uint8_t *down_in = (uint8_t *)calloc((size_t)total_rows * inter / 2, 1);
  uint8_t *down_in_scale =
      (uint8_t *)calloc((size_t)num_expert_local * m_scale_pad * skp_i, 1);
  oracle_grouped_gemm(gate_up, input, gate_up_w, seqlens, cu_seqlens, input_scale,
                      gate_up_ws, num_expert_local, 2 * inter, hidden, m_scale_pad, NULL);
  oracle_act_mul_and_quant(down_in, down_in_scale, gate_up, seqlens, cu_seqlens,
                           num_expert_local, m_scale_pad, inter);
  oracle_grouped_gemm(output, down_in, down_w, seqlens, cu_seqlens, down_in_scale,
                      down_ws, num_expert_local, hidden, inter, m_scale_pad, NULL);
  free(gate_up);
  free(down_in);
  free(down_in_scale);
}

/* src/fused_moe/fused_moe.cu:25-74: route -> expert_moe -> weighted reduce.
 * topk_pos_out / seqlens_out / cu_seqlens_out receive the routing result
 * (any may be NULL). */
ORACLE_API void oracle_fused_moe(uint16_t *output, const uint8_t *input,
                                 const uint8_t *input_scale, const uint8_t *gate_up_w,
                                 const uint8_t *gate_up_ws, const uint8_t *down_w,
                                 const uint8_t *down_ws, const int *topk_ids,
                                 const float *topk_scale, const uint16_t *shared_output,
                                 int num_tokens, int hidden, int inter, int num_topk,
                                 int num_expert_local, int rank_ep, int input_scale_m_pad,
                                 int *topk_pos_out, int *seqlens_out, int *cu_seqlens_out) {
  int total = num_tokens * num_topk;
  int m_pad = (total + 127) / 128 * 128;
  int skp_h = oracle_scale_k_padded(hidden);
  uint8_t *gin, *gscale;
  int *pos, *seqlens, *cu;
  uint16_t *down_out;
  if (m_pad < 128) m_pad = 128;
  gin = (uint8_t *)calloc((size_t)total * hidden / 2, 1);
  gscale = (uint8_t *)calloc((size_t)num_expert_local * m_pad * skp_h, 1);
  pos = (int *)calloc((size_t)total, sizeof(int));
  seqlens = (int *)calloc((size_t)num_expert_local, sizeof(int));
  cu = (int *)calloc((size_t)num_expert_local + 1, sizeof(int));
  down_out = (uint16_t *)calloc((size_t)total * hidden, 2);
  oracle_count_and_gather(gin, gscale, input, input_scale, topk_ids, pos, seqlens, cu,
                          num_tokens, hidden, num_topk, num_expert_local, rank_ep,
                          input_scale_m_pad, m_pad);
  if (cu[num_expert_local] > 0)
    oracle_expert_moe(down_out, gin, gscale, gate_up_w, gate_up_ws, down_w, down_ws,
                      seqlens, cu, total, hidden, inter, num_expert_local, m_pad);
  oracle_reduce(output, down_out, pos, topk_scale, shared_output, num_tokens, hidden,
                num_topk);
  if (topk_pos_out) memcpy(topk_pos_out, pos, (size_t)total * sizeof(int));
  if (seqlens_out) memcpy(seqlens_out, seqlens, (size_t)num_expert_local * sizeof(int));
  if (cu_seqlens_out) memcpy(cu_seqlens_out, cu, ((size_t)num_expert_local + 1) * sizeof(int));
  free(gin);
  free(gscale);
  free(pos);
  free(seqlens);
  free(cu);
  free(down_out);
}

/* Router step in front of the fused MoE. The reference library has no such function (its
 * entry points take topk_ids / topk_weights as inputs; its tests build them by hand,
 * tests/python/test_fused_moe.py:60-75); the DeepSeek-shaped configuration defines it: sigmoid
 * scores, the num_topk largest per token (ties to the lower expert id), weights = score / sum of
 * the selected scores. score = 1 / (1 + exp(-logit)) with oracle_expf, the sum taken in
 * selection order - the operation sequence of the CUDA kernel. */
ORACLE_API void oracle_router_topk(int *topk_ids, float *topk_weights, const float *logits,
                                   int num_tokens, int num_experts, int num_topk) {
  int t;
#pragma omp parallel for schedule(static)
  for (t = 0; t < num_tokens; ++t) {
    float *score = (float *)malloc((size_t)num_experts * sizeof(float));
    float sum = 0.0f;
    int e, r;
    for (e = 0; e < num_experts; ++e)
      score[e] = 1.0f / (1.0f + oracle_expf(-logits[(int64_t)t * num_experts + e]));
    for (r = 0; r < num_topk; ++r) {
      int best = -1;
      for (e = 0; e < num_experts; ++e)
        if (score[e] >= 0.0f && (best < 0 || score[e] > score[best])) best = e;
      topk_ids[t * num_topk + r] = best;
      topk_weights[t * num_topk + r] = best >= 0 ? score[best] : 0.0f;
      if (best >= 0) {
        sum = r == 0 ? score[best] : sum + score[best];
        score[best] = -1.0f;
      }
    }
    for (r = 0; r < num_topk; ++r) topk_weights[t * num_topk + r] = topk_weights[t * num_topk + r] / sum;
    free(score);
  }
}

/* src/fused_moe/fused_moe.cu:76-95 and python/sm120_nvfp4/__init__.py:245-269 */
ORACLE_API uint64_t oracle_expert_moe_workspace_size(int total_rows, int hidden, int inter,
                                                     int num_expert_local, int m_scale_pad) {
  uint64_t total = 0;
  uint64_t sizes[7];
  int i;
  (void)hidden;
  sizes[0] = (uint64_t)total_rows * inter * 2 * 2;
  sizes[1] = (uint64_t)total_rows * inter / 2;
  sizes[2] = (uint64_t)num_expert_local * m_scale_pad * oracle_scale_k_padded(inter);
  sizes[3] = (uint64_t)(num_expert_local * 3 + 2) * 128;
  sizes[4] = sizes[3];
  sizes[5] = (uint64_t)num_expert_local * 4;
  sizes[6] = (uint64_t)(num_expert_local + 1) * 4;
  for (i = 0; i < 7; ++i) {
    total = (total + 255) / 256 * 256;
    total += sizes[i];
  }
  return (total + 255) / 256 * 256;
}

/* Default-path selector: src/gemm/gemm_dispatch.cu:44-56 with the shape rule
 * of src/gemm/specialized/m128_gemm.cu:384-393. 0 generic, 1 M128 split-K 4,
 * 2 M256 split-K 2. */
ORACLE_API int oracle_gemm_path(int m, int n, int k) {
  int ok = n > 0 && k > 0 && (k % 32) == 0 && (n % 8) == 0;
  int tiles_k = (k + 127) / 128;
  if (m == 128 && ok && 4 <= tiles_k) return 1;
  if (m == 256 && ok && 2 <= tiles_k) return 2;
  return 0;
}

ORACLE_API uint64_t oracle_gemm_workspace_size(int m, int n, int k) {
  int path = oracle_gemm_path(m, n, k);
  if (path == 1) return (uint64_t)4 * m * n * 4;
  if (path == 2) return (uint64_t)2 * m * n * 4;
  return 0;
}

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Thread count of the next parallel loops. A launcher that pins OMP_NUM_THREADS=1 for its
 * worker processes (torchrun does) would otherwise make the timed CPU baseline single-threaded. */
ORACLE_API void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
