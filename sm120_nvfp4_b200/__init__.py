"""B200 (sm_100a) drop-in for the hot path of the sm120_nvfp4 Python package.

The functions below have the names, arguments and error behaviour of the reference's
python/sm120_nvfp4/__init__.py (gemm, cute_gemm, cutlass_gemm, grouped_gemm, fused_moe,
quantize_expert, expert_moe, expert_moe_workspace_bytes, scale_k_padded, scale_a_elements,
scale_b_elements) and are also registered as torch.ops.sm120_nvfp4.* with the reference's
schemas. They validate like the reference's bindings (bindings/gemm_ops.cu,
bindings/grouped_gemm_ops.cpp, bindings/fused_moe_ops.cpp), allocate outputs and scratch
with torch, and call the hand-written sm_100a kernels through the C ABI declared in
include/b200_nvfp4.h on torch's current stream. torch is used for memory and streams only.
"""
from __future__ import annotations

from .ops import (HostGemm, autotune_gemm, autotune_grouped_gemm, clear_tuned_tiles, cute_gemm, cutlass_gemm,
                  expert_moe, expert_moe_workspace_bytes, fused_moe, gemm, grouped_gemm, pack_weights,
                  quantize_expert, router_topk, scale_a_elements, scale_b_elements, scale_k_padded, tuned_tile)

__all__ = [
    "expert_moe",
    "expert_moe_workspace_bytes",
    "fused_moe",
    "cute_gemm",
    "cutlass_gemm",
    "gemm",
    "grouped_gemm",
    "quantize_expert",
    "scale_k_padded",
    "scale_a_elements",
    "scale_b_elements",
    # not in the reference package: the callers either side of the routed layer
    "router_topk",
    "pack_weights",
    # host-memory operands, copies overlapped with the arithmetic
    "HostGemm",
    # shape-keyed tile table
    "autotune_gemm",
    "autotune_grouped_gemm",
    "tuned_tile",
    "clear_tuned_tiles",
]
