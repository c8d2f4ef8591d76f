"""ctypes binding of the C ABI in include/b200_nvfp4.h.

There is no fallback: if the shared library is missing and cannot be built, importing the
ops raises. The library is built in-tree by sm120_nvfp4_b200.build.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_LIB_PATH = _PKG / "libb200_nvfp4.so"
_lib = None

STATUS_SUCCESS = 0
STATUS_INVALID_ARGUMENT = 1
STATUS_UNSUPPORTED_DEVICE = 2
STATUS_INSUFFICIENT_WORKSPACE = 3
STATUS_NOT_SUPPORTED = 4
STATUS_CUDA_ERROR = 6

vp = C.c_void_p
ci = C.c_int

_SIGNATURES = {
    "b200_nvfp4_status_string": (C.c_char_p, [ci]),
    "b200_nvfp4_gemm_path_string": (C.c_char_p, [ci]),
    "b200_nvfp4_gemm_path": (ci, [ci, ci, ci]),
    "b200_nvfp4_gemm_workspace_bytes": (C.c_size_t, [ci, ci, ci]),
    "b200_nvfp4_gemm": (ci, [ci, ci, ci, ci, vp, vp, vp, vp, vp, ci, vp]),
    "b200_nvfp4_gemm_splitk": (ci, [ci, ci, ci, ci, vp, vp, vp, vp, vp, vp, C.c_size_t, vp]),
    "b200_nvfp4_gemm_splitk_cluster": (ci, [ci, ci, ci, ci, vp, vp, vp, vp, vp, vp]),
    "b200_nvfp4_gemm_splitk_static_max_elements": (C.c_size_t, []),
    "b200_nvfp4_gemm_splitk_static": (ci, [ci, ci, ci, ci, vp, vp, vp, vp, vp, vp]),
    "b200_nvfp4_gemm_host": (ci, [ci, ci, ci] + [vp] * 10 + [ci, ci, vp]),
    "b200_nvfp4_gemm_auto": (ci, [ci, ci, ci, vp, vp, vp, vp, vp, vp, C.c_size_t, vp]),
    "b200_nvfp4_grouped_gemm": (ci, [vp] * 10 + [ci] * 7 + [vp, vp]),
    "b200_nvfp4_moe_count_and_gather": (ci, [vp] * 8 + [ci] * 8 + [vp]),
    "b200_nvfp4_moe_act_mul_and_quant": (ci, [vp] * 5 + [ci] * 5 + [vp]),
    "b200_nvfp4_moe_quantize_expert": (ci, [vp] * 5 + [ci] * 6 + [vp]),
    "b200_nvfp4_moe_quantize_expert_gather": (ci, [vp] * 6 + [ci] * 6 + [vp]),
    "b200_nvfp4_moe_route": (ci, [vp] * 4 + [ci] * 4 + [vp]),
    "b200_nvfp4_moe_scatter_rows": (ci, [vp] * 3 + [ci] * 3 + [vp]),
    "b200_nvfp4_moe_gather_rows": (ci, [vp] * 3 + [ci] * 2 + [vp]),
    "b200_nvfp4_moe_reduce": (ci, [vp] * 5 + [ci] * 4 + [vp]),
    "b200_nvfp4_fused_moe": (ci, [vp] * 23 + [ci] * 9 + [vp]),
    "b200_nvfp4_expert_moe_workspace_bytes": (C.c_size_t, [ci] * 5),
    "b200_nvfp4_moe_router_topk": (ci, [vp, vp, vp, ci, ci, ci, vp]),
    "b200_nvfp4_grouped_gemm_swiglu_quant": (ci, [vp] * 10 + [ci] * 7 + [vp]),
    "b200_nvfp4_ep_record_bytes": (C.c_size_t, [ci, ci]),
    "b200_nvfp4_ep_dest_ranks": (ci, [vp, vp, ci, ci, ci, ci, vp]),
    "b200_nvfp4_ep_pack_rows": (ci, [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, vp]),
    "b200_nvfp4_ep_unpack_rows": (ci, [vp, vp, vp, vp, vp, ci, ci, ci, vp]),
    "b200_nvfp4_ep_dispatch_p2p": (ci, [vp, vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, vp]),
    "b200_nvfp4_ep_unpack_slots": (ci, [vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp]),
    "b200_nvfp4_ep_barrier_p2p": (ci, [vp, ci, ci, ci, C.c_longlong, vp]),
    "b200_nvfp4_ep_reduce_return_p2p_columns": (ci, [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, vp]),
    "b200_nvfp4_grouped_gemm_columns": (ci, [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp, ci, ci, vp]),
    "b200_nvfp4_ep_publish_p2p": (ci, [vp, ci, ci, ci, ci, vp]),
    "b200_nvfp4_ep_unpack_slots_ready": (ci, [vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp, ci, C.c_longlong, vp]),
    "b200_nvfp4_ep_sum_p2p": (ci, [vp, vp, vp, ci, ci, ci, ci, vp, ci, C.c_longlong, vp]),
    "b200_nvfp4_ep_return_p2p": (ci, [vp, vp, vp, ci, ci, ci, ci, vp]),
    "b200_nvfp4_ep_reduce_return_p2p": (ci, [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, vp]),
    "b200_nvfp4_expert_moe": (ci, [vp] * 10 + [C.c_size_t] + [ci] * 5 + [vp]),
    "b200_nvfp4_device_error": (ci, [C.POINTER(ci)]),
    "b200_nvfp4_set_tile_n": (ci, [ci]),
    "b200_nvfp4_tune_set": (ci, [ci, ci, ci, ci, ci, ci, ci]),
    "b200_nvfp4_tune_get": (ci, [ci, ci, ci, ci, ci, ci]),
    "b200_nvfp4_tune_clear": (None, []),
    "b200_nvfp4_last_launch_tile": (ci, []),
    "b200_nvfp4_set_fused_gate_up": (ci, [ci]),
    "b200_nvfp4_silu_f16": (ci, [vp, vp, ci, vp]),
    "b200_nvfp4_set_wait_limit": (ci, [C.c_longlong, ci]),
    "b200_nvfp4_launch_count": (C.c_longlong, []),
}


def exported_symbols():
    """Names every entry point include/b200_nvfp4.h declares."""
    return sorted(_SIGNATURES)


def lib():
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            from . import build as _build
            _build.build()
        L = C.CDLL(str(_LIB_PATH))
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError here = the library lacks a declared symbol
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = L
    return _lib


def status_string(status: int) -> str:
    return lib().b200_nvfp4_status_string(status).decode()


def check(status: int, what: str) -> None:
    if status != STATUS_SUCCESS:
        raise RuntimeError(f"{what} failed: {status_string(status)}")


def device_error() -> int:
    """Reads and clears the device-side error word (synchronises)."""
    code = ci(0)
    check(lib().b200_nvfp4_device_error(C.byref(code)), "b200_nvfp4_device_error")
    return code.value


def launch_count() -> int:
    return int(lib().b200_nvfp4_launch_count())
