"""numpy/ctypes front end of the CPU oracle (nvfp4_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke entry and by the
CPU-baseline leg of bench.py - never by the shipped package.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from . import build as _build

_HERE = Path(__file__).resolve().parent
_lib = None
_ref = None

u8p = C.POINTER(C.c_uint8)
u16p = C.POINTER(C.c_uint16)
i32p = C.POINTER(C.c_int)
f32p = C.POINTER(C.c_float)


def lib():
    global _lib
    if _lib is None:
        so = _HERE / "liboracle.so"
        src = _HERE / "nvfp4_oracle.c"
        if not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
            _build.build_oracle()
        L = C.CDLL(str(so))
        L.oracle_e2m1_decode.restype = C.c_float
        L.oracle_e2m1_decode.argtypes = [C.c_uint8]
        L.oracle_e2m1_encode.restype = C.c_uint8
        L.oracle_e2m1_encode.argtypes = [C.c_float]
        L.oracle_ue4m3_decode.restype = C.c_float
        L.oracle_ue4m3_decode.argtypes = [C.c_uint8]
        L.oracle_ue4m3_encode.restype = C.c_uint8
        L.oracle_ue4m3_encode.argtypes = [C.c_float]
        L.oracle_f32_to_f16.restype = C.c_uint16
        L.oracle_f32_to_f16.argtypes = [C.c_float]
        L.oracle_f16_to_f32.restype = C.c_float
        L.oracle_f16_to_f32.argtypes = [C.c_uint16]
        L.oracle_f32_to_bf16.restype = C.c_uint16
        L.oracle_f32_to_bf16.argtypes = [C.c_float]
        L.oracle_scale_k_padded.restype = C.c_int
        L.oracle_scale_k_padded.argtypes = [C.c_int]
        L.oracle_sf_offset.restype = C.c_int64
        L.oracle_sf_offset.argtypes = [C.c_int, C.c_int, C.c_int]
        L.oracle_expf.restype = C.c_float
        L.oracle_expf.argtypes = [C.c_float]
        L.oracle_silu.restype = C.c_float
        L.oracle_silu.argtypes = [C.c_float]
        L.oracle_expert_moe_workspace_size.restype = C.c_uint64
        L.oracle_expert_moe_workspace_size.argtypes = [C.c_int] * 5
        L.oracle_gemm_path.restype = C.c_int
        L.oracle_gemm_path.argtypes = [C.c_int] * 3
        L.oracle_gemm_workspace_size.restype = C.c_uint64
        L.oracle_gemm_workspace_size.argtypes = [C.c_int] * 3
        L.oracle_num_threads.restype = C.c_int
        L.oracle_set_num_threads.restype = None
        L.oracle_set_num_threads.argtypes = [C.c_int]
        for name in ("oracle_quantize_rows_f32", "oracle_gemm_sampled", "oracle_gemm",
                     "oracle_grouped_gemm", "oracle_splitk_reduce", "oracle_count_and_gather",
                     "oracle_act_mul_and_quant", "oracle_quantize_expert", "oracle_reduce",
                     "oracle_expert_moe", "oracle_fused_moe", "oracle_router_topk"):
            getattr(L, name).restype = None
        _lib = L
    return _lib


def ref():
    """The reference-derived checker (oracle/_ref), or None where it is not built."""
    global _ref
    if _ref is None:
        so = _build.build_ref()
        if so is None or not Path(so).exists():
            return None
        R = C.CDLL(str(so))
        R.ref_sfa_offset.restype = C.c_int64
        R.ref_sfa_offset.argtypes = [C.c_int] * 4
        R.ref_sfb_offset.restype = C.c_int64
        R.ref_sfb_offset.argtypes = [C.c_int] * 4
        R.ref_sfa_group_elements.restype = C.c_int64
        R.ref_sfa_group_elements.argtypes = [C.c_int] * 2
        for n in ("ref_cutlass_ue4m3_encode", "ref_cutlass_e2m1_encode", "ref_cuda_e2m1_encode",
                  "ref_cuda_e4m3_encode"):
            getattr(R, n).restype = C.c_uint8
            getattr(R, n).argtypes = [C.c_float]
        for n in ("ref_cutlass_ue4m3_decode", "ref_cutlass_e2m1_decode"):
            getattr(R, n).restype = C.c_float
            getattr(R, n).argtypes = [C.c_uint8]
        _ref = R
    return _ref


def set_threads(n: int) -> int:
    """Use n OpenMP threads from now on (e.g. all host cores under a launcher that exported
    OMP_NUM_THREADS=1); returns the count in effect."""
    lib().oracle_set_num_threads(int(n))
    return int(lib().oracle_num_threads())


def _p(a, t):
    return None if a is None else a.ctypes.data_as(t)


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


def scale_k_padded(k: int) -> int:
    return ((k + 15) // 16 + 3) // 4 * 4


def scale_region_bytes(rows: int, k: int) -> int:
    return ((rows + 127) // 128 * 128) * scale_k_padded(k)


def sf_offsets(rows: np.ndarray, kblocks: np.ndarray, k: int) -> np.ndarray:
    """Vectorised closed form of oracle_sf_offset."""
    rows = np.asarray(rows, dtype=np.int64)
    kb = np.asarray(kblocks, dtype=np.int64)
    kt = scale_k_padded(k) // 4
    return ((rows // 128) * kt + kb // 4) * 512 + (rows % 32) * 16 + ((rows % 128) // 32) * 4 + kb % 4


def quantize_rows(x: np.ndarray):
    """FP32 [rows,k] -> (packed uint8 [rows,k/2], scale region uint8)."""
    x = _c(x, np.float32)
    rows, k = x.shape
    packed = np.empty((rows, k // 2), np.uint8)
    scales = np.empty(scale_region_bytes(rows, k), np.uint8)
    lib().oracle_quantize_rows_f32(_p(x, f32p), rows, k, _p(packed, u8p), _p(scales, u8p))
    return packed, scales


def gemm(a, b, sfa, sfb, alpha: float = 1.0):
    """Returns (C fp32, C fp16-as-uint16) for packed A [m,k/2], B [n,k/2]."""
    a, b, sfa, sfb = (_c(t, np.uint8) for t in (a, b, sfa, sfb))
    m, n, k = a.shape[0], b.shape[0], a.shape[1] * 2
    c32 = np.empty((m, n), np.float32)
    c16 = np.empty((m, n), np.uint16)
    lib().oracle_gemm(m, n, k, _p(a, u8p), _p(b, u8p), _p(sfa, u8p), _p(sfb, u8p),
                      C.c_float(alpha), _p(c32, f32p), _p(c16, u16p))
    return c32, c16.view(np.float16)


def gemm_sampled(a, b, sfa, sfb, rows, cols, alpha: float = 1.0):
    a, b, sfa, sfb = (_c(t, np.uint8) for t in (a, b, sfa, sfb))
    m, n, k = a.shape[0], b.shape[0], a.shape[1] * 2
    rows = _c(rows, np.int32)
    cols = _c(cols, np.int32)
    out = np.empty((len(rows), len(cols)), np.float32)
    lib().oracle_gemm_sampled(m, n, k, _p(a, u8p), _p(b, u8p), _p(sfa, u8p), _p(sfb, u8p),
                              _p(rows, i32p), len(rows), _p(cols, i32p), len(cols),
                              C.c_float(alpha), _p(out, f32p))
    return out


def grouped_gemm(x, w, seqlens, cu_seqlens, x_scale, w_scale, m_scale_pad, group_alpha=None,
                 y=None):
    x, w, x_scale, w_scale = (_c(t, np.uint8) for t in (x, w, x_scale, w_scale))
    seqlens = _c(seqlens, np.int32)
    cu_seqlens = _c(cu_seqlens, np.int32)
    g, n, k = w.shape[0], w.shape[1], w.shape[2] * 2
    if y is None:
        y = np.zeros((x.shape[0], n), np.uint16)
    else:
        y = y.view(np.uint16)
    alpha = None if group_alpha is None else _c(group_alpha, np.float32)
    lib().oracle_grouped_gemm(_p(y, u16p), _p(x, u8p), _p(w, u8p), _p(seqlens, i32p),
                              _p(cu_seqlens, i32p), _p(x_scale, u8p), _p(w_scale, u8p), g, n, k,
                              m_scale_pad, _p(alpha, f32p))
    return y.view(np.float16)


def splitk_reduce(partial):
    partial = _c(partial, np.float32)
    splits = partial.shape[0]
    numel = int(np.prod(partial.shape[1:]))
    out = np.empty(partial.shape[1:], np.uint16)
    lib().oracle_splitk_reduce(_p(partial, f32p), splits, C.c_int64(numel), _p(out, u16p))
    return out.view(np.float16)


def count_and_gather(x, x_scale, topk_ids, num_expert_local, rank_ep, input_scale_m_pad,
                     grouped_scale_m_pad):
    x = _c(x, np.uint8)
    x_scale = _c(x_scale, np.uint8)
    topk_ids = _c(topk_ids, np.int32)
    t, topk = topk_ids.shape
    hidden = x.shape[1] * 2
    skp = scale_k_padded(hidden)
    gin = np.zeros((t * topk, hidden // 2), np.uint8)
    gscale = np.empty((num_expert_local, grouped_scale_m_pad * skp), np.uint8)
    pos = np.empty((t, topk), np.int32)
    seqlens = np.empty(num_expert_local, np.int32)
    cu = np.empty(num_expert_local + 1, np.int32)
    lib().oracle_count_and_gather(_p(gin, u8p), _p(gscale, u8p), _p(x, u8p), _p(x_scale, u8p),
                                  _p(topk_ids, i32p), _p(pos, i32p), _p(seqlens, i32p),
                                  _p(cu, i32p), t, hidden, topk, num_expert_local, rank_ep,
                                  input_scale_m_pad, grouped_scale_m_pad)
    return gin, gscale, pos, seqlens, cu


def act_mul_and_quant(gate_up, seqlens, cu_seqlens, m_scale_pad):
    gate_up = np.ascontiguousarray(gate_up).view(np.uint16)
    rows, two_i = gate_up.shape
    inter = two_i // 2
    seqlens = _c(seqlens, np.int32)
    cu_seqlens = _c(cu_seqlens, np.int32)
    e = len(seqlens)
    out = np.zeros((rows, inter // 2), np.uint8)
    scale = np.empty((e, m_scale_pad * scale_k_padded(inter)), np.uint8)
    lib().oracle_act_mul_and_quant(_p(out, u8p), _p(scale, u8p), _p(gate_up, u16p),
                                   _p(seqlens, i32p), _p(cu_seqlens, i32p), e, m_scale_pad, inter)
    return out, scale


def quantize_expert(x_u16, seqlens, cu_seqlens, m_scale_pad, is_bf16):
    x = np.ascontiguousarray(x_u16).view(np.uint16)
    rows, hidden = x.shape
    seqlens = _c(seqlens, np.int32)
    cu_seqlens = _c(cu_seqlens, np.int32)
    e = len(seqlens)
    out = np.zeros((rows, hidden // 2), np.uint8)
    scale = np.empty((e, m_scale_pad * scale_k_padded(hidden)), np.uint8)
    lib().oracle_quantize_expert(_p(out, u8p), _p(scale, u8p), _p(x, u16p), _p(seqlens, i32p),
                                 _p(cu_seqlens, i32p), e, hidden, m_scale_pad, int(bool(is_bf16)))
    return out, scale


def reduce(down_output, topk_pos, topk_scale, shared_output=None):
    down = np.ascontiguousarray(down_output).view(np.uint16)
    pos = _c(topk_pos, np.int32)
    w = _c(topk_scale, np.float32)
    t, topk = pos.shape
    hidden = down.shape[1]
    shared = None if shared_output is None else np.ascontiguousarray(shared_output).view(np.uint16)
    out = np.empty((t, hidden), np.uint16)
    lib().oracle_reduce(_p(out, u16p), _p(down, u16p), _p(pos, i32p), _p(w, f32p),
                        _p(shared, u16p), t, hidden, topk)
    return out.view(np.float16)


def expert_moe(x, x_scale, gate_up_w, gate_up_ws, down_w, down_ws, seqlens, cu_seqlens,
               m_scale_pad):
    x, x_scale, gate_up_w, gate_up_ws, down_w, down_ws = (
        _c(t, np.uint8) for t in (x, x_scale, gate_up_w, gate_up_ws, down_w, down_ws))
    seqlens = _c(seqlens, np.int32)
    cu_seqlens = _c(cu_seqlens, np.int32)
    rows, hidden = x.shape[0], x.shape[1] * 2
    e, inter = gate_up_w.shape[0], gate_up_w.shape[1] // 2
    out = np.zeros((rows, hidden), np.uint16)
    lib().oracle_expert_moe(_p(out, u16p), _p(x, u8p), _p(x_scale, u8p), _p(gate_up_w, u8p),
                            _p(gate_up_ws, u8p), _p(down_w, u8p), _p(down_ws, u8p),
                            _p(seqlens, i32p), _p(cu_seqlens, i32p), rows, hidden, inter, e,
                            m_scale_pad)
    return out.view(np.float16)


def fused_moe(x, x_scale, gate_up_w, gate_up_ws, down_w, down_ws, topk_ids, topk_weights,
              shared_output=None, rank_ep=0):
    x, x_scale, gate_up_w, gate_up_ws, down_w, down_ws = (
        _c(t, np.uint8) for t in (x, x_scale, gate_up_w, gate_up_ws, down_w, down_ws))
    ids = _c(topk_ids, np.int32)
    w = _c(topk_weights, np.float32)
    t, topk = ids.shape
    hidden = x.shape[1] * 2
    e, inter = gate_up_w.shape[0], gate_up_w.shape[1] // 2
    in_m_pad = x_scale.size // scale_k_padded(hidden)
    shared = None if shared_output is None else np.ascontiguousarray(shared_output).view(np.uint16)
    out = np.empty((t, hidden), np.uint16)
    pos = np.empty((t, topk), np.int32)
    seqlens = np.empty(e, np.int32)
    cu = np.empty(e + 1, np.int32)
    lib().oracle_fused_moe(_p(out, u16p), _p(x, u8p), _p(x_scale, u8p), _p(gate_up_w, u8p),
                           _p(gate_up_ws, u8p), _p(down_w, u8p), _p(down_ws, u8p), _p(ids, i32p),
                           _p(w, f32p), _p(shared, u16p), t, hidden, inter, topk, e, rank_ep,
                           in_m_pad, _p(pos, i32p), _p(seqlens, i32p), _p(cu, i32p))
    return out.view(np.float16), pos, seqlens, cu


def router_topk(logits, num_topk: int):
    logits = _c(logits, np.float32)
    t, e = logits.shape
    ids = np.empty((t, num_topk), np.int32)
    w = np.empty((t, num_topk), np.float32)
    lib().oracle_router_topk(_p(ids, i32p), _p(w, f32p), _p(logits, f32p), t, e, num_topk)
    return ids, w


E2M1_LEVELS = np.array([0., .5, 1., 1.5, 2., 3., 4., 6., -0., -.5, -1., -1.5, -2., -3., -4., -6.],
                       np.float32)


def decode_packed(packed: np.ndarray) -> np.ndarray:
    """uint8 [..., k/2] -> float32 [..., k] (low nibble = even k)."""
    packed = np.asarray(packed, np.uint8)
    lo = E2M1_LEVELS[packed & 15]
    hi = E2M1_LEVELS[packed >> 4]
    return np.stack((lo, hi), -1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)


def decode_ue4m3(b: np.ndarray) -> np.ndarray:
    b = np.asarray(b, np.uint8).astype(np.int32)
    e = (b >> 3) & 15
    m = b & 7
    v = np.where(e == 0, m * 2.0 ** -9, (1 + m / 8.0) * 2.0 ** (e - 7.0))
    return v.astype(np.float32)
