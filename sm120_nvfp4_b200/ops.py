"""Validation, allocation and dispatch for the torch-facing operators.

Mirrors the reference's binding layer: bindings/gemm_ops.cu:43-164,
bindings/grouped_gemm_ops.cpp:16-204 and bindings/fused_moe_ops.cpp:46-495. The checks and
their messages follow those files (TORCH_CHECK -> RuntimeError here); the compute goes to
the C ABI. One deliberate difference: grouped_gemm does not copy seqlens / cu_seqlens to the
host to validate them (grouped_gemm_ops.cpp:113-135 forces a device synchronisation there).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib

_FP4X2 = getattr(torch, "float4_e2m1fn_x2", None)


def scale_k_padded(k: int) -> int:
    return ((k + 15) // 16 + 3) // 4 * 4


def scale_a_elements(m: int, n: int, k: int) -> int:
    del n
    return ((m + 127) // 128 * 128) * scale_k_padded(k)


def scale_b_elements(m: int, n: int, k: int) -> int:
    del m
    return ((n + 127) // 128 * 128) * scale_k_padded(k)


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _is_packed(t: torch.Tensor) -> bool:
    return t.dtype == torch.uint8 or (_FP4X2 is not None and t.dtype == _FP4X2)


def _check_cuda_contig(t: torch.Tensor, device: torch.device, name: str) -> None:
    _check(t.is_cuda, f"{name} must be a CUDA tensor")
    _check(t.device == device, f"{name} must be on the same CUDA device as input")
    _check(t.is_contiguous(), f"{name} must be contiguous")


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# --------------------------------------------------------------------------- GEMM


def _gemm_common(a, b, sfa, sfb, mode: str) -> torch.Tensor:
    _check(a.is_cuda and b.is_cuda and sfa.is_cuda and sfb.is_cuda, "all inputs must be CUDA tensors")
    device = a.device
    for t, name in ((a, "a"), (b, "b"), (sfa, "sfa"), (sfb, "sfb")):
        _check_cuda_contig(t, device, name)
    _check(_is_packed(a) and _is_packed(b), "a and b must be float4_e2m1fn_x2 or packed uint8")
    _check(a.dtype == b.dtype, "a and b must use the same packed storage dtype")
    _check(sfa.dtype == torch.uint8 and sfb.dtype == torch.uint8,
           "sfa and sfb must contain raw UE4M3 bytes (uint8)")
    _check(a.dim() == 2 and b.dim() == 2, "a and b must be two-dimensional packed matrices")
    _check(a.size(1) == b.size(1), "a and b must share the packed K dimension")
    m, n, k = a.size(0), b.size(0), a.size(1) * 2
    _check(m > 0 and n > 0 and k > 0, "M, N and K must be positive")
    _check(k % 32 == 0, "K must be a multiple of 32")
    _check(n % 8 == 0, "N must be a multiple of 8")
    _check(sfa.numel() == scale_a_elements(m, n, k), "sfa has the wrong physical size")
    _check(sfb.numel() == scale_b_elements(m, n, k), "sfb has the wrong physical size")
    out = torch.empty((m, n), dtype=torch.float16, device=device)
    L = _lib.lib()
    with torch.cuda.device(device):
        stream = _stream(device)
        if mode == "auto":
            ws_bytes = L.b200_nvfp4_gemm_workspace_bytes(m, n, k)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device) if ws_bytes else None
            status = L.b200_nvfp4_gemm_auto(m, n, k, a.data_ptr(), b.data_ptr(), sfa.data_ptr(),
                                            sfb.data_ptr(), out.data_ptr(), _ptr(ws), ws_bytes, stream)
        else:
            status = L.b200_nvfp4_gemm(1, m, n, k, a.data_ptr(), b.data_ptr(), sfa.data_ptr(),
                                       sfb.data_ptr(), out.data_ptr(), 0, stream)
    _check(status == 0, f"NVFP4 GEMM failed: {_lib.status_string(status)}")
    return out


def gemm(a: torch.Tensor, b: torch.Tensor, sfa: torch.Tensor, sfb: torch.Tensor) -> torch.Tensor:
    """Compute GEMM with M=128/M=256 specialization and generic fallback."""
    return _gemm_common(a, b, sfa, sfb, "auto")


def cute_gemm(a: torch.Tensor, b: torch.Tensor, sfa: torch.Tensor, sfb: torch.Tensor) -> torch.Tensor:
    """Run the generic persistent kernel (no split-K)."""
    return _gemm_common(a, b, sfa, sfb, "generic")


def cutlass_gemm(a: torch.Tensor, b: torch.Tensor, sfa: torch.Tensor, sfb: torch.Tensor) -> torch.Tensor:
    """Name kept from the reference, where it runs a CUTLASS comparison kernel; this library
    ships none, so it runs the generic kernel."""
    return _gemm_common(a, b, sfa, sfb, "generic")


class HostGemm:
    """GEMM on operands that live in (page-locked) host memory: `run(a, b, sfa, sfb, out)` uploads A and B
    in chunks, computes each block of C as soon as its two chunks have landed and copies it home while
    later chunks still arrive (`b200_nvfp4_gemm_host`). The object owns the device scratch for one
    problem size; the result is complete once the current stream has been synchronised. Not in the
    reference, whose operators take device tensors only."""

    def __init__(self, m: int, n: int, k: int, device=None, block_rows: int = 0, block_cols: int = 0):
        _check(m > 0 and n > 0 and k > 0 and k % 32 == 0 and n % 8 == 0,
               "M, N, K must be positive, K % 32 == 0 and N % 8 == 0")
        self.m, self.n, self.k = m, n, k
        self.block_rows, self.block_cols = block_rows, block_cols
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        u8 = dict(dtype=torch.uint8, device=self.device)
        self._a = torch.empty((m, k // 2), **u8)
        self._b = torch.empty((n, k // 2), **u8)
        self._sfa = torch.empty(scale_a_elements(m, n, k), **u8)
        self._sfb = torch.empty(scale_b_elements(m, n, k), **u8)
        self._c = torch.empty((m, n), dtype=torch.float16, device=self.device)

    def run(self, a: torch.Tensor, b: torch.Tensor, sfa: torch.Tensor, sfb: torch.Tensor,
            out: torch.Tensor = None) -> torch.Tensor:
        m, n, k = self.m, self.n, self.k
        for t, name in ((a, "a"), (b, "b"), (sfa, "sfa"), (sfb, "sfb")):
            _check(not t.is_cuda and t.is_contiguous(), f"{name} must be a contiguous host tensor")
        _check(_is_packed(a) and _is_packed(b) and tuple(a.shape) == (m, k // 2) and tuple(b.shape) == (n, k // 2),
               "a must be packed [M, K/2] and b packed [N, K/2]")
        _check(sfa.dtype == torch.uint8 and sfb.dtype == torch.uint8 and sfa.numel() == self._sfa.numel()
               and sfb.numel() == self._sfb.numel(), "sfa / sfb have the wrong dtype or physical size")
        if out is None:
            out = torch.empty((m, n), dtype=torch.float16).pin_memory()
        _check(not out.is_cuda and out.is_contiguous() and out.dtype == torch.float16 and tuple(out.shape) == (m, n),
               "out must be a contiguous float16 host tensor [M, N]")
        L = _lib.lib()
        with torch.cuda.device(self.device):
            status = L.b200_nvfp4_gemm_host(m, n, k, a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(),
                                            out.data_ptr(), self._a.data_ptr(), self._b.data_ptr(),
                                            self._sfa.data_ptr(), self._sfb.data_ptr(), self._c.data_ptr(),
                                            self.block_rows, self.block_cols, _stream(self.device))
        _check(status == 0, f"NVFP4 host GEMM failed: {_lib.status_string(status)}")
        return out


# ------------------------------------------------------------------- grouped GEMM


def _grouped_gemm_op(x, weight, seqlens, cu_seqlens, x_scale, weight_scale, num_seq_per_group_avg,
                     output=None, tma_desc=None, group_alpha=None) -> torch.Tensor:
    _check(x.is_cuda, "x must be a CUDA tensor")
    device = x.device
    for t, name in ((x, "x"), (weight, "weight"), (seqlens, "seqlens"), (cu_seqlens, "cu_seqlens"),
                    (x_scale, "x_scale"), (weight_scale, "weight_scale")):
        _check_cuda_contig(t, device, name)
    _check(_is_packed(x) and _is_packed(weight), "x and weight must be float4_e2m1fn_x2 or packed uint8")
    _check(x.dtype == weight.dtype, "x and weight must use the same packed storage dtype")
    _check(x_scale.dtype == torch.uint8 and weight_scale.dtype == torch.uint8,
           "scale tensors must contain raw UE4M3 bytes (uint8)")
    _check(seqlens.dtype == torch.int32 and cu_seqlens.dtype == torch.int32,
           "seqlens and cu_seqlens must be int32")
    _check(x.dim() == 2 and weight.dim() == 3, "x must be [rows, K/2] and weight [groups, N, K/2]")
    groups, n = weight.size(0), weight.size(1)
    m, k = x.size(0), x.size(1) * 2
    _check(weight.size(2) == x.size(1), "x and weight must share the packed K dimension")
    _check(0 < groups <= 256, "number of groups must be in [1, 256]")
    _check(m > 0 and k % 32 == 0 and n % 8 == 0, "rows must be positive, K % 32 == 0 and N % 8 == 0")
    _check(seqlens.numel() == groups and cu_seqlens.numel() == groups + 1,
           "seqlens / cu_seqlens lengths are inconsistent with the number of groups")
    skp = scale_k_padded(k)
    _check(x_scale.dim() == 2 and x_scale.size(0) == groups and x_scale.size(1) % skp == 0,
           "x_scale must have physical shape [groups, m_scale_pad * scale_k_padded(K)]")
    m_scale_pad = x_scale.size(1) // skp
    _check(m_scale_pad >= 128 and m_scale_pad % 128 == 0,
           "x_scale must reserve a 128-row-aligned region per group")
    _check(weight_scale.dim() == 2 and weight_scale.size(0) == groups and
           weight_scale.size(1) == scale_b_elements(1, n, k), "weight_scale has an invalid physical shape")
    if output is not None:
        _check_cuda_contig(output, device, "output")
        _check(output.dtype == torch.float16 and tuple(output.shape) == (m, n),
               "output must be contiguous FP16 [rows, N]")
        out = output
    else:
        out = torch.empty((m, n), dtype=torch.float16, device=device)
    if tma_desc is not None:
        _check_cuda_contig(tma_desc, device, "tma_desc")
        _check(tma_desc.dtype == torch.uint8 and tma_desc.numel() >= (3 * groups + 2) * 128 and
               tma_desc.data_ptr() % 128 == 0, "tma_desc must be 128-byte aligned and hold (3G+2)*128 bytes")
    tiles = torch.empty(groups, dtype=torch.int32, device=device)
    cu_tiles = torch.empty(groups + 1, dtype=torch.int32, device=device)
    if group_alpha is not None:
        _check_cuda_contig(group_alpha, device, "group_alpha")
        _check(group_alpha.dtype == torch.float32 and group_alpha.numel() == groups,
               "group_alpha must be float32 [groups]")
    with torch.cuda.device(device):
        status = _lib.lib().b200_nvfp4_grouped_gemm(
            out.data_ptr(), x.data_ptr(), weight.data_ptr(), seqlens.data_ptr(), cu_seqlens.data_ptr(),
            x_scale.data_ptr(), weight_scale.data_ptr(), _ptr(tma_desc), tiles.data_ptr(),
            cu_tiles.data_ptr(), groups, m, n, k, m_scale_pad, int(num_seq_per_group_avg), 1,
            _ptr(group_alpha), _stream(device))
    _check(status == 0, f"group_gemm_nvfp4 launch failed: {_lib.status_string(status)}")
    return out


def grouped_gemm(x, weight, seqlens, cu_seqlens, x_scale, weight_scale, *, output=None,
                 workspace=None, group_alpha=None) -> torch.Tensor:
    """Run expert-major grouped NVFP4 GEMMs with a single persistent launch.

    group_alpha (optional FP32 [groups]) is an extension: a per-group multiplier applied to
    the FP32 accumulator before the FP16 rounding.
    """
    groups = int(weight.shape[0])
    average_rows = int(x.shape[0]) // groups if groups else 0
    if group_alpha is None:
        return torch.ops.sm120_nvfp4.grouped_gemm(x, weight, seqlens, cu_seqlens, x_scale,
                                                  weight_scale, average_rows, output, workspace)
    return _grouped_gemm_op(x, weight, seqlens, cu_seqlens, x_scale, weight_scale, average_rows,
                            output, workspace, group_alpha)


# ---------------------------------------------------------------------- fused MoE


def _check_moe_weights(x, gate_up_weight, gate_up_weight_scale, down_weight, down_weight_scale,
                       hidden_size):
    num_expert_local = gate_up_weight.size(0)
    gate_up_size = gate_up_weight.size(1)
    _check(0 < num_expert_local <= 256, "num_expert_local must be in [1, 256]")
    _check(gate_up_size > 0 and gate_up_size % 2 == 0, "gate_up_weight.size(1) must be 2 * intermediate_size")
    inter = gate_up_size // 2
    _check(hidden_size % 32 == 0 and inter % 32 == 0,
           "hidden_size and intermediate_size must be multiples of 32")
    _check(gate_up_weight.size(2) == x.size(1), "input and gate_up_weight must share packed hidden_size/2")
    _check(tuple(down_weight.shape) == (num_expert_local, hidden_size, inter // 2),
           "down_weight shape must be [num_expert_local, hidden_size, intermediate_size/2]")
    expected_gate = ((gate_up_size + 127) // 128 * 128) * scale_k_padded(hidden_size)
    expected_down = ((hidden_size + 127) // 128 * 128) * scale_k_padded(inter)
    _check(tuple(gate_up_weight_scale.shape) == (num_expert_local, expected_gate),
           f"gate_up_weight_scale must have physical shape [{num_expert_local}, {expected_gate}]")
    _check(tuple(down_weight_scale.shape) == (num_expert_local, expected_down),
           f"down_weight_scale must have physical shape [{num_expert_local}, {expected_down}]")
    return num_expert_local, inter


def _fused_moe_op(x, x_scale, gate_up_weight, gate_up_weight_scale, down_weight, down_weight_scale,
                  topk_ids, topk_scale, shared_output, rank_ep, num_expert_total, output) -> torch.Tensor:
    _check(x.is_cuda, "input must be a CUDA tensor")
    device = x.device
    for t, name in ((x, "input"), (x_scale, "input_scale"), (gate_up_weight, "gate_up_weight"),
                    (gate_up_weight_scale, "gate_up_weight_scale"), (down_weight, "down_weight"),
                    (down_weight_scale, "down_weight_scale"), (topk_ids, "topk_ids"),
                    (topk_scale, "topk_scale")):
        _check_cuda_contig(t, device, name)
    _check(_is_packed(x) and _is_packed(gate_up_weight) and _is_packed(down_weight),
           "input, gate_up_weight and down_weight must be float4_e2m1fn_x2 or packed uint8")
    _check(x.dtype == gate_up_weight.dtype == down_weight.dtype,
           "all packed E2M1 tensors must use the same storage dtype")
    _check(x_scale.dtype == torch.uint8 and gate_up_weight_scale.dtype == torch.uint8 and
           down_weight_scale.dtype == torch.uint8,
           "all NVFP4 scale tensors must contain raw UE4M3 bytes (uint8)")
    _check(topk_ids.dtype == torch.int32, "topk_ids must be int32")
    _check(topk_scale.dtype == torch.float32, "topk_scale must be float32")
    _check(x.dim() == 2, "input must have packed shape [num_tokens, hidden_size/2]")
    _check(gate_up_weight.dim() == 3 and down_weight.dim() == 3, "weights must be three-dimensional")
    _check(topk_ids.dim() == 2 and topk_scale.dim() == 2, "topk_ids and topk_scale must be two-dimensional")
    _check(topk_ids.shape == topk_scale.shape, "topk_ids and topk_scale must have the same shape")
    _check(topk_ids.size(0) == x.size(0), "topk routing tensors and input must share num_tokens")
    num_tokens, hidden_size, num_topk = x.size(0), x.size(1) * 2, topk_ids.size(1)
    _check(num_tokens > 0, "num_tokens must be in the positive int32 range")
    _check(0 < num_topk <= 128, "num_topk must be in [1, 128]")
    num_expert_local, inter = _check_moe_weights(x, gate_up_weight, gate_up_weight_scale, down_weight,
                                                 down_weight_scale, hidden_size)
    _check(num_expert_total > 0, "num_expert_total must be in the positive int32 range")
    _check(rank_ep >= 0, "rank_ep must be a non-negative int32 value")
    _check(rank_ep * num_expert_local + num_expert_local <= num_expert_total,
           "rank_ep and num_expert_local select experts outside num_expert_total")
    total = num_tokens * num_topk
    _check(total <= 2 ** 31 - 1, "num_tokens * num_topk exceeds the int32 range")
    m_pad = max(128, (total + 127) // 128 * 128)
    skp_h, skp_i = scale_k_padded(hidden_size), scale_k_padded(inter)
    _check(x_scale.numel() % skp_h == 0, "input_scale physical size is incompatible with hidden_size")
    in_m_pad = x_scale.numel() // skp_h
    _check(in_m_pad >= num_tokens and in_m_pad % 128 == 0,
           "input_scale must use a 128-row-aligned block-scaled SFA region")
    if output is not None:
        _check_cuda_contig(output, device, "output")
        _check(output.dtype == torch.float16 and tuple(output.shape) == (num_tokens, hidden_size),
               "output must be contiguous FP16 [num_tokens, hidden_size]")
        result = output
    else:
        result = torch.empty((num_tokens, hidden_size), dtype=torch.float16, device=device)
    if shared_output is not None:
        _check_cuda_contig(shared_output, device, "shared_output")
        _check(shared_output.dtype == torch.float16 and tuple(shared_output.shape) == (num_tokens, hidden_size),
               "shared_output must be contiguous FP16 [num_tokens, hidden_size]")
    u8 = dict(dtype=torch.uint8, device=device)
    i32 = dict(dtype=torch.int32, device=device)
    f16 = dict(dtype=torch.float16, device=device)
    gate_up_input = torch.empty((total, hidden_size // 2), **u8)
    gate_up_input_scale = torch.empty((num_expert_local, m_pad * skp_h), **u8)
    gate_up_output = torch.empty((total, 2 * inter), **f16)
    down_input = torch.empty((total, inter // 2), **u8)
    down_input_scale = torch.empty((num_expert_local, m_pad * skp_i), **u8)
    down_output = torch.empty((total, hidden_size), **f16)
    topk_pos = torch.empty((num_tokens, num_topk), **i32)
    seqlens = torch.empty(num_expert_local, **i32)
    cu_seqlens = torch.empty(num_expert_local + 1, **i32)
    tiles = torch.empty(num_expert_local, **i32)
    cu_tiles = torch.empty(num_expert_local + 1, **i32)
    with torch.cuda.device(device):
        status = _lib.lib().b200_nvfp4_fused_moe(
            result.data_ptr(), x.data_ptr(), x_scale.data_ptr(), gate_up_input.data_ptr(),
            gate_up_input_scale.data_ptr(), gate_up_output.data_ptr(), gate_up_weight.data_ptr(),
            gate_up_weight_scale.data_ptr(), None, down_input.data_ptr(), down_input_scale.data_ptr(),
            down_output.data_ptr(), down_weight.data_ptr(), down_weight_scale.data_ptr(), None,
            topk_ids.data_ptr(), topk_scale.data_ptr(), topk_pos.data_ptr(), seqlens.data_ptr(),
            cu_seqlens.data_ptr(), tiles.data_ptr(), cu_tiles.data_ptr(), _ptr(shared_output),
            num_tokens, hidden_size, inter, num_topk, int(num_expert_total), num_expert_local,
            int(rank_ep), in_m_pad, m_pad, _stream(device))
    _check(status == 0, f"fuse_moe_nvfp4 launch failed: {_lib.status_string(status)}")
    return result


def fused_moe(x, x_scale, gate_up_weight, gate_up_weight_scale, down_weight, down_weight_scale,
              topk_ids, topk_weights, *, shared_output=None, ep_rank: int = 0,
              num_experts: Optional[int] = None, output=None) -> torch.Tensor:
    """Run routing, two grouped GEMMs, activation/quantization and reduction."""
    if num_experts is None:
        num_experts = int(gate_up_weight.shape[0])
    return torch.ops.sm120_nvfp4.fused_moe(x, x_scale, gate_up_weight, gate_up_weight_scale,
                                           down_weight, down_weight_scale, topk_ids, topk_weights,
                                           shared_output, ep_rank, num_experts, output)


def _quantize_expert_op(x, seqlens, cu_seqlens, scale_m_pad, output, output_scale
                        ) -> Tuple[torch.Tensor, torch.Tensor]:
    _check(x.is_cuda, "input must be a CUDA tensor")
    device = x.device
    for t, name in ((x, "input"), (seqlens, "seqlens"), (cu_seqlens, "cu_seqlens")):
        _check_cuda_contig(t, device, name)
    _check(x.dtype in (torch.float16, torch.bfloat16), "input must be float16 or bfloat16")
    _check(seqlens.dtype == torch.int32 and cu_seqlens.dtype == torch.int32,
           "seqlens and cu_seqlens must be int32")
    _check(x.dim() == 2 and seqlens.dim() == 1 and cu_seqlens.dim() == 1,
           "input must be [rows, hidden] and prefix tensors must be 1D")
    rows, hidden = x.shape
    e = seqlens.size(0)
    _check(rows > 0 and hidden > 0 and hidden % 32 == 0,
           "rows must be positive and hidden_size a positive multiple of 32")
    _check(0 < e <= 256 and cu_seqlens.size(0) == e + 1,
           "prefix tensor lengths are inconsistent with local experts")
    _check(scale_m_pad >= 128 and scale_m_pad % 128 == 0, "scale_m_pad must be a positive multiple of 128")
    if output is not None:
        _check_cuda_contig(output, device, "output")
        _check(output.dtype == torch.uint8 and tuple(output.shape) == (rows, hidden // 2),
               "output must be uint8 [rows, hidden/2]")
        packed = output
    else:
        packed = torch.empty((rows, hidden // 2), dtype=torch.uint8, device=device)
    scale_elems = scale_m_pad * scale_k_padded(hidden)
    if output_scale is not None:
        _check_cuda_contig(output_scale, device, "output_scale")
        _check(output_scale.dtype == torch.uint8 and tuple(output_scale.shape) == (e, scale_elems),
               "output_scale has an invalid physical SFA shape")
        scales = output_scale
    else:
        scales = torch.empty((e, scale_elems), dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        status = _lib.lib().b200_nvfp4_moe_quantize_expert(
            packed.data_ptr(), scales.data_ptr(), x.data_ptr(), seqlens.data_ptr(), cu_seqlens.data_ptr(),
            e, rows, hidden, int(scale_m_pad), int(x.dtype == torch.bfloat16), 1, _stream(device))
    _check(status == 0, f"quantize_expert_nvfp4 launch failed: {_lib.status_string(status)}")
    return packed, scales


def quantize_expert(x, seqlens, cu_seqlens, *, scale_m_pad: Optional[int] = None, output=None,
                    output_scale=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantize an expert-major FP16/BF16 matrix to packed NVFP4."""
    if scale_m_pad is None:
        scale_m_pad = max(128, ((int(x.shape[0]) + 127) // 128) * 128)
    return torch.ops.sm120_nvfp4.quantize_expert(x, seqlens, cu_seqlens, scale_m_pad, output, output_scale)


def expert_moe_workspace_bytes(total_rows: int, hidden_size: int, intermediate_size: int,
                               num_experts: int, scale_m_pad: int) -> int:
    """Return bytes required by :func:`expert_moe` reusable scratch storage."""
    del hidden_size
    alignment = 256
    total = 0
    for size in (total_rows * intermediate_size * 4, total_rows * intermediate_size // 2,
                 num_experts * scale_m_pad * scale_k_padded(intermediate_size),
                 (num_experts * 3 + 2) * 128, (num_experts * 3 + 2) * 128, num_experts * 4,
                 (num_experts + 1) * 4):
        total = (total + alignment - 1) // alignment * alignment + size
    return (total + alignment - 1) // alignment * alignment


def _expert_moe_op(x, x_scale, gate_up_weight, gate_up_weight_scale, down_weight, down_weight_scale,
                   seqlens, cu_seqlens, output, workspace) -> torch.Tensor:
    _check(x.is_cuda, "input must be a CUDA tensor")
    device = x.device
    for t, name in ((x, "input"), (x_scale, "input_scale"), (gate_up_weight, "gate_up_weight"),
                    (gate_up_weight_scale, "gate_up_weight_scale"), (down_weight, "down_weight"),
                    (down_weight_scale, "down_weight_scale"), (seqlens, "seqlens"),
                    (cu_seqlens, "cu_seqlens")):
        _check_cuda_contig(t, device, name)
    _check(_is_packed(x) and _is_packed(gate_up_weight) and _is_packed(down_weight),
           "input and weights must use packed E2M1 storage")
    _check(x.dtype == gate_up_weight.dtype == down_weight.dtype,
           "input and weights must use the same packed storage dtype")
    _check(x_scale.dtype == torch.uint8 and gate_up_weight_scale.dtype == torch.uint8 and
           down_weight_scale.dtype == torch.uint8, "all scale tensors must contain raw UE4M3 bytes")
    _check(seqlens.dtype == torch.int32 and cu_seqlens.dtype == torch.int32,
           "seqlens and cu_seqlens must be int32")
    _check(x.dim() == 2 and x_scale.dim() == 2 and gate_up_weight.dim() == 3 and
           gate_up_weight_scale.dim() == 2 and down_weight.dim() == 3 and down_weight_scale.dim() == 2 and
           seqlens.dim() == 1 and cu_seqlens.dim() == 1, "expert_moe received tensors with invalid ranks")
    rows, hidden = x.size(0), x.size(1) * 2
    _check(rows > 0 and hidden > 0, "rows, hidden size and local expert count must be positive")
    e, inter = _check_moe_weights(x, gate_up_weight, gate_up_weight_scale, down_weight,
                                  down_weight_scale, hidden)
    _check(seqlens.size(0) == e and cu_seqlens.size(0) == e + 1,
           "prefix tensor lengths must match local expert count")
    skp_h = scale_k_padded(hidden)
    _check(x_scale.size(0) == e and x_scale.size(1) % skp_h == 0, "input_scale has an invalid physical SFA shape")
    m_pad = x_scale.size(1) // skp_h
    _check(m_pad >= 128 and m_pad % 128 == 0, "input_scale must reserve a 128-row-aligned region per expert")
    if output is not None:
        _check_cuda_contig(output, device, "output")
        _check(output.dtype == torch.float16 and tuple(output.shape) == (rows, hidden),
               "output must be float16 [rows, hidden]")
        result = output
    else:
        result = torch.empty((rows, hidden), dtype=torch.float16, device=device)
    L = _lib.lib()
    required = L.b200_nvfp4_expert_moe_workspace_bytes(rows, hidden, inter, e, m_pad)
    if workspace is not None:
        _check_cuda_contig(workspace, device, "workspace")
        _check(workspace.dtype == torch.uint8 and workspace.numel() >= required,
               "workspace must be a sufficiently large contiguous uint8 tensor")
        scratch = workspace
    else:
        scratch = torch.empty(required, dtype=torch.uint8, device=device)
    _check(scratch.data_ptr() % 256 == 0, "workspace data pointer must be 256-byte aligned")
    with torch.cuda.device(device):
        status = L.b200_nvfp4_expert_moe(
            result.data_ptr(), x.data_ptr(), x_scale.data_ptr(), gate_up_weight.data_ptr(),
            gate_up_weight_scale.data_ptr(), down_weight.data_ptr(), down_weight_scale.data_ptr(),
            seqlens.data_ptr(), cu_seqlens.data_ptr(), scratch.data_ptr(), scratch.numel(), rows, hidden,
            inter, e, m_pad, _stream(device))
    _check(status == 0, f"expert_moe_nvfp4 launch failed: {_lib.status_string(status)}")
    return result


def expert_moe(x, x_scale, gate_up_weight, gate_up_weight_scale, down_weight, down_weight_scale,
               seqlens, cu_seqlens, *, output=None, workspace=None) -> torch.Tensor:
    """Compute already-routed expert-major activations without local re-routing."""
    return torch.ops.sm120_nvfp4.expert_moe(x, x_scale, gate_up_weight, gate_up_weight_scale, down_weight,
                                            down_weight_scale, seqlens, cu_seqlens, output, workspace)


# ------------------------------------------------------- torch.ops registration
# Same schemas as bindings/gemm_ops.cu:157-164, bindings/grouped_gemm_ops.cpp:197-204 and
# bindings/fused_moe_ops.cpp:473-495. When an output tensor is passed the reference returns
# that very tensor; torch's Python-registered operators may not return an input alias, so the
# raw torch.ops.* entries return a fresh view of it (same data_ptr), as the wrappers above do.

_LIBRARY = torch.library.Library("sm120_nvfp4", "FRAGMENT")
_LIBRARY.define("gemm(Tensor a, Tensor b, Tensor sfa, Tensor sfb) -> Tensor")
_LIBRARY.define("cute_gemm(Tensor a, Tensor b, Tensor sfa, Tensor sfb) -> Tensor")
_LIBRARY.define("cutlass_gemm(Tensor a, Tensor b, Tensor sfa, Tensor sfb) -> Tensor")
_LIBRARY.define("grouped_gemm(Tensor x, Tensor weight, Tensor seqlens, Tensor cu_seqlens, Tensor x_scale, "
                "Tensor w_scale, int num_seq_per_group_avg, Tensor? output, Tensor? tma_desc) -> Tensor")
_LIBRARY.define("fused_moe(Tensor input, Tensor input_scale, Tensor gate_up_weight, "
                "Tensor gate_up_weight_scale, Tensor down_weight, Tensor down_weight_scale, "
                "Tensor topk_ids, Tensor topk_scale, Tensor? shared_output, int rank_ep, "
                "int num_expert_total, Tensor? output) -> Tensor")
_LIBRARY.define("quantize_expert(Tensor input, Tensor seqlens, Tensor cu_seqlens, int scale_m_pad, "
                "Tensor? output, Tensor? output_scale) -> (Tensor, Tensor)")
_LIBRARY.define("expert_moe(Tensor input, Tensor input_scale, Tensor gate_up_weight, "
                "Tensor gate_up_weight_scale, Tensor down_weight, Tensor down_weight_scale, "
                "Tensor seqlens, Tensor cu_seqlens, Tensor? output, Tensor? workspace) -> Tensor")


def _fresh(result: torch.Tensor, *maybe_aliases) -> torch.Tensor:
    for t in maybe_aliases:
        if t is not None and result is t:
            return result.view(result.shape)
    return result


def _grouped_impl(x, weight, seqlens, cu_seqlens, x_scale, w_scale, avg, output, tma_desc):
    return _fresh(_grouped_gemm_op(x, weight, seqlens, cu_seqlens, x_scale, w_scale, avg, output, tma_desc),
                  output)


def _fused_impl(x, xs, gw, gws, dw, dws, ids, w, shared, rank_ep, num_total, output):
    return _fresh(_fused_moe_op(x, xs, gw, gws, dw, dws, ids, w, shared, rank_ep, num_total, output), output)


def _quant_impl(x, seqlens, cu_seqlens, scale_m_pad, output, output_scale):
    packed, scales = _quantize_expert_op(x, seqlens, cu_seqlens, scale_m_pad, output, output_scale)
    return _fresh(packed, output), _fresh(scales, output_scale)


def _expert_impl(x, xs, gw, gws, dw, dws, seqlens, cu_seqlens, output, workspace):
    return _fresh(_expert_moe_op(x, xs, gw, gws, dw, dws, seqlens, cu_seqlens, output, workspace), output)


_LIBRARY.impl("gemm", lambda a, b, sfa, sfb: _gemm_common(a, b, sfa, sfb, "auto"), "CUDA")
_LIBRARY.impl("cute_gemm", lambda a, b, sfa, sfb: _gemm_common(a, b, sfa, sfb, "generic"), "CUDA")
_LIBRARY.impl("cutlass_gemm", lambda a, b, sfa, sfb: _gemm_common(a, b, sfa, sfb, "generic"), "CUDA")
_LIBRARY.impl("grouped_gemm", _grouped_impl, "CUDA")
_LIBRARY.impl("fused_moe", _fused_impl, "CUDA")
_LIBRARY.impl("quantize_expert", _quant_impl, "CUDA")
_LIBRARY.impl("expert_moe", _expert_impl, "CUDA")


# ------------------------------------------------------------------------------------------
# Callers either side of the routed layer. Neither exists in the reference package (its router
# step and its weight conversion are left to the caller); both run this library's CUDA kernels.

def router_topk(logits: torch.Tensor, num_topk: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Router step: FP32 logits [T, E] -> (topk_ids int32 [T, k], topk_weights float32 [T, k]).

    score = sigmoid(logit); the k largest per token, ties to the lower expert id; weights are the
    selected scores divided by their sum. The outputs are what fused_moe takes as topk_ids /
    topk_weights.
    """
    _check(logits.is_cuda and logits.dim() == 2 and logits.dtype == torch.float32 and logits.is_contiguous(),
           "logits must be a contiguous float32 CUDA tensor [num_tokens, num_experts]")
    t, e = logits.shape
    _check(t > 0 and 0 < num_topk <= e <= 4096, "need num_tokens > 0 and 0 < num_topk <= num_experts <= 4096")
    ids = torch.empty((t, num_topk), dtype=torch.int32, device=logits.device)
    weights = torch.empty((t, num_topk), dtype=torch.float32, device=logits.device)
    with torch.cuda.device(logits.device):
        status = _lib.lib().b200_nvfp4_moe_router_topk(logits.data_ptr(), ids.data_ptr(), weights.data_ptr(), t, e,
                                                       int(num_topk), _stream(logits.device))
    _check(status == 0, f"router_topk launch failed: {_lib.status_string(status)}")
    return ids, weights


def pack_weights(weight: torch.Tensor, weight_scale: Optional[torch.Tensor] = None, *,
                 global_scale: bool = False):
    """Expert weights [E, N, K] from a checkpoint -> NVFP4 in the layout grouped_gemm / fused_moe expect
    for `weight` / `weight_scale`: (packed E2M1 uint8 [E, N, K/2], UE4M3 scales uint8
    [E, align128(N) * scale_k_padded(K)]), one UE4M3 scale = amax / 6 per 16 values of K, one
    128-row-aligned block-scaled region per expert.

    weight        BF16, FP16, FP32 or FP8 (float8_e4m3fn) values.
    weight_scale  optional FP32 dequantisation scales of an FP8 checkpoint: [E] (per tensor) or
                  [E, ceil(N/128), ceil(K/128)] (128 x 128 blocks); the weight used is value * scale.
    global_scale  False: the reference's convention, a global scale of 1.0. True: a per-expert FP32 scale
                  g = amax / (448 * 6) is divided out first, so that the block scales use UE4M3's whole
                  range whatever the magnitude of the weights; a third tensor g [E] is returned, to be
                  applied to the GEMM output (grouped_gemm's group_alpha / the caller's epilogue).

    BF16 / FP16 inputs without scales go to the row quantiser as they are; everything else is brought to
    FP32 first (FP8 values and the products with FP32 scales are exact or correctly rounded there) and
    quantised from FP32.
    """
    _check(weight.is_cuda and weight.dim() == 3 and weight.is_contiguous(),
           "weight must be a contiguous CUDA tensor [experts, N, K]")
    fp8 = getattr(torch, "float8_e4m3fn", None)
    _check(weight.dtype in (torch.bfloat16, torch.float16, torch.float32) or (fp8 is not None and weight.dtype == fp8),
           "weight must be BF16, FP16, FP32 or float8_e4m3fn")
    e, n, k = weight.shape
    _check(k % 32 == 0, "K must be a multiple of 32")
    dev = weight.device
    direct = weight.dtype in (torch.bfloat16, torch.float16) and weight_scale is None and not global_scale
    if direct:
        w = weight
    else:
        w = weight.to(torch.float32)
        if weight_scale is not None:
            _check(weight_scale.is_cuda and weight_scale.dtype == torch.float32, "weight_scale must be FP32 on the device")
            if weight_scale.dim() == 1:
                _check(weight_scale.shape[0] == e, "per-tensor weight_scale must be [experts]")
                w = w * weight_scale.view(e, 1, 1)
            else:
                nb, kb = (n + 127) // 128, (k + 127) // 128
                _check(tuple(weight_scale.shape) == (e, nb, kb), "block weight_scale must be [experts, ceil(N/128), ceil(K/128)]")
                full = weight_scale.repeat_interleave(128, dim=1)[:, :n].repeat_interleave(128, dim=2)[:, :, :k]
                w = w * full
    alpha = None
    if global_scale:
        amax = w.abs().amax(dim=(1, 2)).to(torch.float32)
        alpha = torch.where(amax > 0, amax / (448.0 * 6.0), torch.ones_like(amax))
        w = w / alpha.view(e, 1, 1)
    w = w.contiguous()
    seqlens = torch.full((e,), n, dtype=torch.int32, device=dev)
    cu = torch.arange(0, (e + 1) * n, n, dtype=torch.int32, device=dev)
    m_pad = (n + 127) // 128 * 128
    if w.dtype == torch.float32:
        packed = torch.empty((e * n, k // 2), dtype=torch.uint8, device=dev)
        scales = torch.empty((e, m_pad * scale_k_padded(k)), dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            status = _lib.lib().b200_nvfp4_moe_quantize_expert(packed.data_ptr(), scales.data_ptr(), w.data_ptr(),
                                                               seqlens.data_ptr(), cu.data_ptr(), e, e * n, k, m_pad, 2,
                                                               1, _stream(dev))
        _check(status == 0, f"quantize_expert_nvfp4 launch failed: {_lib.status_string(status)}")
    else:
        packed, scales = quantize_expert(w.view(e * n, k), seqlens, cu, scale_m_pad=m_pad)
    packed = packed.view(e, n, k // 2)
    return (packed, scales, alpha) if global_scale else (packed, scales)


# ---------------------------------------------------------------------------------- tile table
#
# Not in the reference package (its RTX 5090 tuning is compiled in): times the tile shapes of the
# GEMM kernel on the device for one problem and records the fastest in the library's shape-keyed
# table (b200_nvfp4_tune_set), which the built-in rules then defer to for exactly that problem.

_TILES = (64, 128, 256, 512)      # 128-row tiles of 64 / 128 / 256 columns on one CTA; 512 = 256 x 256 on a CTA pair


def _time_tiles(call, device, candidates, iters: int):
    """Microseconds per call (CUDA events around `iters` back-to-back calls, three warm-up calls
    first) for every candidate tile, forced through b200_nvfp4_set_tile_n."""
    L = _lib.lib()
    times = {}
    try:
        for tile in candidates:
            _check(tile in _TILES, f"tile must be one of {_TILES}")
            _lib.check(L.b200_nvfp4_set_tile_n(tile), "set_tile_n")
            for _ in range(3):
                call()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(torch.cuda.current_stream(device))
            for _ in range(iters):
                call()
            end.record(torch.cuda.current_stream(device))
            end.synchronize()
            times[tile] = start.elapsed_time(end) * 1e3 / iters
    finally:
        L.b200_nvfp4_set_tile_n(0)
    _check(_lib.device_error() == 0, "a kernel reported a timed-out wait while tuning")
    return times


def autotune_gemm(m: int, n: int, k: int, *, batch: int = 1, out_dtype: torch.dtype = torch.float16, device=None,
                  candidates=_TILES, iters: int = 30, install: bool = True) -> dict:
    """Times the dense (batch = 1) or batched NVFP4 GEMM of this shape with every candidate tile on
    random operands and, with install=True, records the fastest for the shape. Returns
    {"best": tile, "us": {tile: microseconds per call}}. Timing only: the result of a GEMM does not
    depend on the tile (tests/test_gpu_determinism.py)."""
    _check(out_dtype in (torch.float16, torch.float32), "out_dtype must be float16 or float32")
    _check(m > 0 and n > 0 and k > 0 and k % 32 == 0 and n % 8 == 0 and batch > 0,
           "M, N, K, batch must be positive, K % 32 == 0 and N % 8 == 0")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    L = _lib.lib()
    f32 = int(out_dtype == torch.float32)
    with torch.cuda.device(device):
        g = torch.Generator(device=device).manual_seed(k * 31 + n)
        a = torch.randint(0, 256, (batch, m, k // 2), dtype=torch.uint8, device=device, generator=g)
        b = torch.randint(0, 256, (batch, n, k // 2), dtype=torch.uint8, device=device, generator=g)
        sfa = torch.randint(0x30, 0x3a, (batch * scale_a_elements(m, n, k),), dtype=torch.uint8, device=device, generator=g)
        sfb = torch.randint(0x30, 0x3a, (batch * scale_b_elements(m, n, k),), dtype=torch.uint8, device=device, generator=g)
        out = torch.empty((batch, m, n), dtype=out_dtype, device=device)
        stream = _stream(device)

        def call():
            _lib.check(L.b200_nvfp4_gemm(batch, m, n, k, a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(),
                                         out.data_ptr(), f32, stream), "gemm")

        times = _time_tiles(call, device, candidates, iters)
    best = min(times, key=times.get)
    if install:
        _lib.check(L.b200_nvfp4_tune_set(batch, m, n, k, f32, 0, best), "tune_set")
    return {"best": best, "us": times}


def autotune_grouped_gemm(seqlens, n: int, k: int, *, device=None, candidates=_TILES, iters: int = 30,
                          install: bool = True) -> dict:
    """The same for the grouped GEMM over groups of `seqlens` rows (a representative split: the table
    is keyed by the number of groups and the total number of rows, the row counts themselves live
    on the device)."""
    counts = [int(c) for c in seqlens]
    _check(len(counts) > 0 and all(c >= 0 for c in counts) and sum(counts) > 0, "seqlens must hold row counts")
    _check(n > 0 and k > 0 and k % 32 == 0 and n % 8 == 0, "N, K must be positive, K % 32 == 0 and N % 8 == 0")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    L = _lib.lib()
    groups, rows = len(counts), sum(counts)
    m_pad = max(128, (max(counts) + 127) // 128 * 128)
    with torch.cuda.device(device):
        g = torch.Generator(device=device).manual_seed(k * 31 + n + groups)
        x = torch.randint(0, 256, (rows, k // 2), dtype=torch.uint8, device=device, generator=g)
        w = torch.randint(0, 256, (groups, n, k // 2), dtype=torch.uint8, device=device, generator=g)
        xs = torch.randint(0x30, 0x3a, (groups * m_pad * scale_k_padded(k),), dtype=torch.uint8, device=device, generator=g)
        ws = torch.randint(0x30, 0x3a, (groups * scale_b_elements(1, n, k),), dtype=torch.uint8, device=device, generator=g)
        seq = torch.tensor(counts, dtype=torch.int32, device=device)
        cu = torch.zeros(groups + 1, dtype=torch.int32, device=device)
        cu[1:] = torch.cumsum(seq, 0)
        out = torch.empty((rows, n), dtype=torch.float16, device=device)
        stream = _stream(device)
        avg = max(1, rows // groups)

        def call():
            _lib.check(L.b200_nvfp4_grouped_gemm(out.data_ptr(), x.data_ptr(), w.data_ptr(), seq.data_ptr(),
                                                 cu.data_ptr(), xs.data_ptr(), ws.data_ptr(), None, None, None, groups,
                                                 rows, n, k, m_pad, avg, 1, None, stream), "grouped_gemm")

        times = _time_tiles(call, device, candidates, iters)
    best = min(times, key=times.get)
    if install:
        _lib.check(L.b200_nvfp4_tune_set(groups, rows, n, k, 0, 1, best), "tune_set")
    return {"best": best, "us": times}


def tuned_tile(rows: int, n: int, k: int, *, groups: int = 1, out_dtype: torch.dtype = torch.float16,
               grouped: bool = False) -> int:
    """The table's tile for a problem (0 = none: the built-in rules apply)."""
    return int(_lib.lib().b200_nvfp4_tune_get(groups, rows, n, k, int(out_dtype == torch.float32), int(grouped)))


def clear_tuned_tiles() -> None:
    _lib.lib().b200_nvfp4_tune_clear()
