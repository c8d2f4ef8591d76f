"""CPU-only checks: the C-ABI library builds, loads and exports every declared symbol, the
host-side dispatcher / size functions agree with the oracle, and the Python surface mirrors
the reference's names. No kernel is launched here."""
import re
from pathlib import Path

import numpy as np
import pytest

import oracle

ROOT = Path(__file__).resolve().parents[1]


def test_library_exports_every_declared_symbol():
    from sm120_nvfp4_b200 import _lib
    L = _lib.lib()
    header = (ROOT / "include" / "b200_nvfp4.h").read_text()
    declared = sorted(set(re.findall(r"\b(b200_nvfp4_[a-z0-9_]+)\s*\(", header)))
    assert declared == _lib.exported_symbols()
    for name in declared:
        assert hasattr(L, name), name


def test_dispatcher_and_workspace_match_oracle():
    from sm120_nvfp4_b200 import _lib
    L = _lib.lib()
    O = oracle.lib()
    cases = [(16, 4096, 8192), (128, 4096, 8192), (256, 4096, 8192), (128, 128, 128), (128, 128, 512),
             (256, 136, 128), (256, 136, 256), (128, 4100, 8192), (128, 4096, 8200), (0, 8, 32), (128, 0, 512)]
    for m, n, k in cases:
        assert L.b200_nvfp4_gemm_path(m, n, k) == O.oracle_gemm_path(m, n, k), (m, n, k)
        assert L.b200_nvfp4_gemm_workspace_bytes(m, n, k) == O.oracle_gemm_workspace_size(m, n, k)
    assert L.b200_nvfp4_gemm_path_string(0) == b"generic_cute"
    assert L.b200_nvfp4_gemm_path_string(1) == b"m128_splitk4"
    assert L.b200_nvfp4_gemm_path_string(2) == b"m256_splitk2"
    assert L.b200_nvfp4_status_string(0) == b"success"
    assert L.b200_nvfp4_status_string(3) == b"workspace is null or too small"
    assert L.b200_nvfp4_status_string(99) == b"unknown status"


def test_expert_moe_workspace_matches_oracle_and_python_mirror():
    import sm120_nvfp4_b200 as pkg
    from sm120_nvfp4_b200 import _lib
    L = _lib.lib()
    O = oracle.lib()
    for args in ((5, 128, 64, 2, 128), (32768, 7168, 2048, 256, 32768), (777, 512, 96, 7, 384)):
        want = O.oracle_expert_moe_workspace_size(*args)
        assert L.b200_nvfp4_expert_moe_workspace_bytes(*args) == want
        assert pkg.expert_moe_workspace_bytes(*args) == want


def test_argument_validation_without_gpu():
    from sm120_nvfp4_b200 import _lib
    L = _lib.lib()
    # invalid shapes / null pointers are rejected before any CUDA call
    assert L.b200_nvfp4_gemm(1, 16, 4096, 8190, 16, 16, 16, 16, 16, 0, None) == 1
    assert L.b200_nvfp4_gemm(1, 16, 4097, 8192, 16, 16, 16, 16, 16, 0, None) == 1
    assert L.b200_nvfp4_gemm(1, 16, 4096, 8192, None, 16, 16, 16, 16, 0, None) == 1
    assert L.b200_nvfp4_gemm(1, 16, 4096, 8192, 24, 16, 16, 16, 16, 0, None) == 1  # misaligned
    assert L.b200_nvfp4_gemm_auto(128, 4096, 8192, 16, 16, 16, 16, 16, None, 0, None) == 3
    assert L.b200_nvfp4_gemm_auto(128, 4096, 8192, 16, 16, 16, 16, 16, 16, 100, None) == 3
    assert L.b200_nvfp4_expert_moe(16, 16, 16, 16, 16, 16, 16, 16, 16, None, 0, 5, 128, 64, 2, 128, None) == 3
    # host-memory GEMM: chunk sizes must be multiples of the 128-row scale atoms; no null pointers
    assert L.b200_nvfp4_gemm_host(256, 256, 128, *([16] * 10), 100, 128, None) == 1
    assert L.b200_nvfp4_gemm_host(256, 256, 128, *([16] * 9), None, 128, 128, None) == 1
    assert L.b200_nvfp4_gemm_host(256, 260, 128, *([16] * 10), 128, 128, None) == 1
    assert L.b200_nvfp4_set_tile_n(48) == 1 and L.b200_nvfp4_set_tile_n(32) == 1 and L.b200_nvfp4_set_tile_n(0) == 0


def test_python_surface_mirrors_reference_names():
    import sm120_nvfp4_b200 as pkg
    import torch
    for name in ("gemm", "cute_gemm", "cutlass_gemm", "grouped_gemm", "fused_moe", "quantize_expert",
                 "expert_moe", "expert_moe_workspace_bytes", "scale_k_padded", "scale_a_elements",
                 "scale_b_elements", "router_topk", "pack_weights", "HostGemm"):
        assert callable(getattr(pkg, name))
    for op in ("gemm", "cute_gemm", "cutlass_gemm", "grouped_gemm", "fused_moe", "quantize_expert", "expert_moe"):
        assert hasattr(torch.ops.sm120_nvfp4, op)
    assert pkg.scale_k_padded(8192) == 512 and pkg.scale_k_padded(7168) == 448 and pkg.scale_k_padded(80) == 8
    assert pkg.scale_a_elements(16, 4096, 8192) == 128 * 512
    assert pkg.scale_b_elements(16, 4096, 8192) == 4096 * 512
    a = torch.zeros((16, 64), dtype=torch.uint8)
    with pytest.raises(RuntimeError):
        pkg.cute_gemm(a, a, a, a)  # CPU tensors are rejected, as by the reference binding


def test_synthetic_data_generators_are_seeded():
    from helpers import dirichlet_counts, randn_quantized, topk_routing
    p1, s1 = randn_quantized(8, 64, 5)
    p2, s2 = randn_quantized(8, 64, 5)
    assert (p1 == p2).all() and (s1 == s2).all()
    ids, w = topk_routing(16, 32, 4, 1)
    assert ids.shape == (16, 4) and np.allclose(w.sum(1), 1.0, atol=1e-6)
    assert all(len(set(r)) == 4 for r in ids.tolist())
    counts, cu = dirichlet_counts(2048, 8, 3)
    assert counts.sum() == 2048 and cu[-1] == 2048


def test_tile_table_is_keyed_by_the_whole_problem():
    # b200_nvfp4_tune_set / _get / _clear: host-side state only, no device needed.
    import sm120_nvfp4_b200 as pkg
    from sm120_nvfp4_b200 import _lib
    L = _lib.lib()
    pkg.clear_tuned_tiles()
    assert pkg.tuned_tile(16, 4096, 8192) == 0
    assert L.b200_nvfp4_tune_set(1, 16, 4096, 8192, 0, 0, 128) == 0
    assert pkg.tuned_tile(16, 4096, 8192) == 128
    # every field of the key matters: rows, N, K, groups, output type, dense against grouped
    assert pkg.tuned_tile(32, 4096, 8192) == 0 and pkg.tuned_tile(16, 4096, 4096) == 0
    assert pkg.tuned_tile(16, 2048, 8192) == 0 and pkg.tuned_tile(16, 4096, 8192, groups=2) == 0
    import torch
    assert pkg.tuned_tile(16, 4096, 8192, out_dtype=torch.float32) == 0
    assert pkg.tuned_tile(16, 4096, 8192, grouped=True) == 0
    assert L.b200_nvfp4_tune_set(1, 16, 4096, 8192, 0, 0, 512) == 0      # overwrite
    assert pkg.tuned_tile(16, 4096, 8192) == 512
    assert L.b200_nvfp4_tune_set(1, 16, 4096, 8192, 0, 0, 0) == 0        # 0 removes
    assert pkg.tuned_tile(16, 4096, 8192) == 0
    for bad in ((0, 16, 64, 64, 0, 0, 64), (1, 0, 64, 64, 0, 0, 64), (1, 16, 64, 64, 0, 0, 96), (1, 16, 64, 64, 0, 0, 1024)):
        assert L.b200_nvfp4_tune_set(*bad) == _lib.STATUS_INVALID_ARGUMENT
    L.b200_nvfp4_tune_set(8, 2048, 4096, 8192, 0, 1, 256)
    pkg.clear_tuned_tiles()
    assert pkg.tuned_tile(2048, 4096, 8192, groups=8, grouped=True) == 0


def test_hand_off_and_window_entry_points_validate_without_gpu():
    # The entry points added for the expert-parallel hand-off and the column-window GEMM reject bad
    # arguments before any CUDA call (dummy non-null pointers, 16-byte aligned).
    import ctypes
    from sm120_nvfp4_b200 import _lib
    L = _lib.lib()
    bad = _lib.STATUS_INVALID_ARGUMENT
    p = 4096
    # column window: start not a multiple of 128, inner window not a multiple of 128, past the end, empty
    for start, count in ((64, 128), (0, 200), (640, 128), (0, 0), (-128, 128)):
        assert L.b200_nvfp4_grouped_gemm_columns(p, p, p, p, p, p, p, 3, 440, 648, 256, 384, 150, None, start, count,
                                                 None) == bad
    table = (ctypes.c_void_p * 2)(p, p)
    assert L.b200_nvfp4_ep_publish_p2p(table, 2, 2, 0, 1, None) == bad          # rank outside the world
    assert L.b200_nvfp4_ep_publish_p2p(table, 0, 65, 0, 1, None) == bad         # more ranks than the flag area holds
    assert L.b200_nvfp4_ep_publish_p2p(table, 0, 2, -1, 1, None) == bad
    assert L.b200_nvfp4_ep_publish_p2p((ctypes.c_void_p * 2)(p, None), 0, 2, 0, 1, None) == bad
    assert L.b200_nvfp4_ep_sum_p2p(p, p, p, 4, 130, 2, 0, p, 1, 0, None) == bad  # hidden not a multiple of 8
    assert L.b200_nvfp4_ep_sum_p2p(p, p, p, 0, 128, 2, 0, p, 1, 0, None) == bad
    assert L.b200_nvfp4_ep_sum_p2p(p, p, p, 4, 128, 2, 0, p + 2, 1, 0, None) == bad   # misaligned ready words
    assert L.b200_nvfp4_ep_sum_p2p(p, p, p, 4, 128, 2, 0, p, 1, -5, None) == bad       # negative limit
    assert L.b200_nvfp4_ep_unpack_slots_ready(p, p, p, p, p, p, 2, 4, 128, 2, p + 1, 1, 0, None) == bad
    assert L.b200_nvfp4_ep_unpack_slots_ready(p, p, p, p, p, p, 2, 4, 128, 2, p, 1, -1, None) == bad
    for start, count in ((4, 64), (0, 0), (0, 132), (128, 64)):
        assert L.b200_nvfp4_ep_reduce_return_p2p_columns(table, p, p, p, p, 0, 2, 4, 128, 2, start, count, None) == bad
