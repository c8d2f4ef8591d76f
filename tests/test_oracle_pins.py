"""Pin the CPU oracle against the reference's golden vectors (CPU only).

Sources of the pins: committed fixtures under tests/golden/ (made from the
reference by tests/golden/make_golden.py), the known answers of the reference's
own tests, and - where the reference checkout is present - the live
reference-derived checker in oracle/_ref.
"""
import math

import numpy as np
import pytest

import oracle


def test_codecs_match_cutlass_and_cuda_host_conversions(golden_dir):
    g = np.load(golden_dir / "codecs.npz")
    L = oracle.lib()
    v = g["value"]
    ue = np.array([L.oracle_ue4m3_encode(float(abs(x))) for x in v], np.uint8)
    # cvt.rn.satfinite.e4m3x2.f32, emulated on the host by the CUDA toolkit
    np.testing.assert_array_equal(ue, g["cuda_e4m3"])
    # CUTLASS's software path agrees everywhere below the saturation point
    finite = np.abs(v) < 448
    np.testing.assert_array_equal(ue[finite], g["cutlass_ue4m3"][finite])
    e2 = np.array([L.oracle_e2m1_encode(float(x)) for x in v], np.uint8)
    np.testing.assert_array_equal(e2, g["cuda_e2m1"])
    np.testing.assert_array_equal(e2, g["cutlass_e2m1"])
    np.testing.assert_array_equal(
        np.array([L.oracle_ue4m3_decode(b) for b in range(0x7f)], np.float32), g["ue4m3_table"])
    np.testing.assert_array_equal(
        np.array([L.oracle_e2m1_decode(b) for b in range(16)], np.float32), g["e2m1_table"])
    np.testing.assert_array_equal(oracle.decode_ue4m3(np.arange(0x7f)), g["ue4m3_table"])


def test_documented_code_points():
    L = oracle.lib()
    # docs/API.md:11 and tests/python/test_gemm.py:42-47
    assert L.oracle_ue4m3_decode(0x38) == 1.0 and L.oracle_ue4m3_decode(0x30) == 0.5
    assert L.oracle_ue4m3_decode(0x7e) == 448.0
    assert L.oracle_ue4m3_decode(0x18) == 0.0625 and L.oracle_ue4m3_decode(0x20) == 0.125
    assert L.oracle_e2m1_decode(0x2) == 1.0 and L.oracle_e2m1_decode(0x1) == 0.5
    assert L.oracle_ue4m3_encode(500.0) == 0x7e and L.oracle_ue4m3_encode(2.0 ** -10) == 0
    # tests/python/test_fused_moe.py:96-101: 1024/6 -> 176, 1024/176 -> 6
    assert L.oracle_ue4m3_decode(L.oracle_ue4m3_encode(1024.0 / 6.0)) == 176.0
    assert L.oracle_e2m1_decode(L.oracle_e2m1_encode(1024.0 / 176.0)) == 6.0
    assert L.oracle_ue4m3_decode(L.oracle_ue4m3_encode(256.0 / 6.0)) == 44.0
    for tie, want in ((0.25, 0.0), (0.75, 1.0), (2.5, 2.0), (5.0, 4.0), (1.25, 1.0), (3.5, 4.0)):
        assert L.oracle_e2m1_decode(L.oracle_e2m1_encode(tie)) == want


def test_half_conversions_match_numpy():
    L = oracle.lib()
    rng = np.random.default_rng(3)
    vals = np.concatenate([rng.normal(size=4000) * 100, np.exp(rng.uniform(-20, 12, 4000)),
                           [0.0, -0.0, 65504.0, 65520.0, 1e9, 2.0 ** -24, 2.0 ** -25, 3 * 2.0 ** -25]]
                          ).astype(np.float32)
    got = np.array([L.oracle_f32_to_f16(float(x)) for x in vals], np.uint16)
    with np.errstate(over="ignore"):
        np.testing.assert_array_equal(got, vals.astype(np.float16).view(np.uint16))
    allh = np.arange(0, 0x7c00, 7, dtype=np.uint16)
    back = np.array([L.oracle_f16_to_f32(int(h)) for h in allh], np.float32)
    np.testing.assert_array_equal(back, allh.view(np.float16).astype(np.float32))


def test_scale_layout_matches_reference_offsets(golden_dir):
    g = np.load(golden_dir / "sf_layout.npz")
    L = oracle.lib()
    for r, kb, m_pad, k, sfa, sfb in zip(g["row"], g["k_block"], g["m_pad"], g["k"], g["sfa"], g["sfb"]):
        off = L.oracle_sf_offset(int(r), int(kb), int(k))
        assert off == sfa == sfb, (r, kb, m_pad, k)
    np.testing.assert_array_equal(oracle.sf_offsets(g["row"][:64], g["k_block"][:64], int(g["k"][0])),
                                  g["sfa"][:64])


def test_scale_layout_matches_live_reference_header():
    R = oracle.ref()
    if R is None:
        pytest.skip("reference checkout not present: oracle/_ref not built")
    L = oracle.lib()
    for m_pad, k in ((128, 128), (256, 80), (384, 7168), (128, 8192), (256, 2048)):
        assert R.ref_sfa_group_elements(m_pad, k) == m_pad * L.oracle_scale_k_padded(k)
        for r in range(0, m_pad, 5):
            for kb in range((k + 15) // 16):
                assert R.ref_sfa_offset(r, kb, m_pad, k) == L.oracle_sf_offset(r, kb, k)
                assert R.ref_sfb_offset(r, kb, m_pad, k) == L.oracle_sf_offset(r, kb, k)


def test_offset_formula_in_reference_moe_test():
    # tests/python/test_fused_moe.py:160-168 (M=K=128)
    L = oracle.lib()
    for row in range(4):
        for kb in range(8):
            want = (kb // 4) * 512 + (row % 32) * 16 + (row // 32) * 4 + (kb % 4)
            assert L.oracle_sf_offset(row, kb, 128) == want


def test_quantizer_matches_reference_torch_restatement(golden_dir):
    g = np.load(golden_dir / "quantizer.npz")
    x = g["input_bf16_bits"]
    rows, hidden = x.shape
    packed, scale = oracle.quantize_expert(x, [rows], [0, rows], 128, True)
    vals = oracle.decode_packed(packed).reshape(rows, hidden // 16, 16)
    rr, kk = np.meshgrid(np.arange(rows), np.arange(hidden // 16), indexing="ij")
    sf = oracle.decode_ue4m3(scale[0][oracle.sf_offsets(rr, kk, hidden)])
    dequant = (vals * sf[..., None]).reshape(rows, hidden)
    np.testing.assert_array_equal(dequant, g["expected_dequant"])


def test_all_ones_gemm_gives_k():
    # tests/python/test_gemm.py:39-68,102-134
    for m, n, k in ((16, 128, 128), (64, 136, 128), (129, 136, 128), (128, 128, 512)):
        a = np.full((m, k // 2), 0x22, np.uint8)
        b = np.full((n, k // 2), 0x22, np.uint8)
        sfa = np.full(oracle.scale_region_bytes(m, k), 0x38, np.uint8)
        sfb = np.full(oracle.scale_region_bytes(n, k), 0x38, np.uint8)
        c32, c16 = oracle.gemm(a, b, sfa, sfb)
        assert (c16 == np.float16(k)).all() and (c32 == k).all()


def test_dyadic_random_payload_gemm(golden_dir):
    g = np.load(golden_dir / "dyadic_gemm.npz")
    n, k = 256, 512
    for m in (7, 128, 256):
        sfa = np.full(oracle.scale_region_bytes(m, k), 0x18, np.uint8)
        sfb = np.full(oracle.scale_region_bytes(n, k), 0x20, np.uint8)
        _, c16 = oracle.gemm(g[f"a_{m}"], g[f"b_{m}"], sfa, sfb)
        np.testing.assert_array_equal(c16, g[f"expected_{m}"])


def test_grouped_gemm_empty_experts_and_tails(golden_dir):
    g = np.load(golden_dir / "dyadic_gemm.npz")
    groups, rows, n, k, pad = 4, 257, 128, 128, 256
    codes = g["gcodes"]
    xs = np.repeat(codes[:, None], pad * oracle.scale_k_padded(k), 1)
    ws = np.repeat(codes[::-1][:, None], oracle.scale_region_bytes(n, k), 1)
    for idx in range(2):
        counts = g[f"gcounts_{idx}"]
        cu = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
        y = oracle.grouped_gemm(g["gx"], g["gw"], counts, cu, xs, ws, pad)
        np.testing.assert_array_equal(y, g[f"gexpected_{idx}"])


def test_cpp_reference_gemm_case():
    # tests/cpp/test_gemm.cu:74-80,216-234: sparse 0/1 payloads, SFA=2, SFB=1
    m, n, k = 16, 64, 8192
    kk = np.arange(k)
    a_val = (((np.arange(m)[:, None] + kk[None]) & 7) == 0).astype(np.float32)
    b_val = (((kk[None] + 3 * np.arange(n)[:, None]) & 15) == 0).astype(np.float32)
    code = lambda v: (v * 2).astype(np.uint8)  # 1.0 -> nibble 2
    a = (code(a_val)[:, 0::2] | (code(a_val)[:, 1::2] << 4)).astype(np.uint8)
    b = (code(b_val)[:, 0::2] | (code(b_val)[:, 1::2] << 4)).astype(np.uint8)
    sfa = np.full(oracle.scale_region_bytes(m, k), oracle.lib().oracle_ue4m3_encode(2.0), np.uint8)
    sfb = np.full(oracle.scale_region_bytes(n, k), oracle.lib().oracle_ue4m3_encode(1.0), np.uint8)
    c32, _ = oracle.gemm(a, b, sfa, sfb)
    np.testing.assert_array_equal(c32, (a_val * 2.0) @ b_val.T)


def test_dispatcher_table():
    # tests/cpp/test_gemm.cu:95-103
    L = oracle.lib()
    table = ((16, 4096, 8192, 0, 0), (128, 4096, 8192, 1, 4 * 128 * 4096 * 4),
             (256, 4096, 8192, 2, 2 * 256 * 4096 * 4), (128, 128, 128, 0, 0))
    for m, n, k, path, ws in table:
        assert L.oracle_gemm_path(m, n, k) == path
        assert L.oracle_gemm_workspace_size(m, n, k) == ws


def _moe_case():
    tokens, experts, hidden, inter = 4, 2, 128, 64
    x = np.full((tokens, hidden // 2), 0x11, np.uint8)
    gw = np.full((experts, 2 * inter, hidden // 2), 0x11, np.uint8)
    dw = np.full((experts, hidden, inter // 2), 0x11, np.uint8)
    xs = np.full(128 * 8, 0x38, np.uint8)
    gs = np.full((experts, 128 * 8), 0x38, np.uint8)
    ds = np.full((experts, 128 * 4), 0x38, np.uint8)
    return tokens, experts, hidden, x, xs, gw, gs, dw, ds


def test_moe_uniform_known_answer():
    # tests/python/test_fused_moe.py:55-101
    tokens, experts, hidden, x, xs, gw, gs, dw, ds = _moe_case()
    ids = np.array([[0, 1], [1, 0], [0, 1], [1, 0]], np.int32)
    w = np.array([[0.25, 0.75], [0.6, 0.4], [0.5, 0.5], [0.2, 0.8]], np.float32)
    shared = np.full((tokens, hidden), 2.0, np.float16)
    out, pos, seqlens, cu = oracle.fused_moe(x, xs, gw, gs, dw, ds, ids, w, shared)
    assert (out.astype(np.float32) == 33792.0).all()
    assert seqlens.tolist() == [4, 4] and cu.tolist() == [0, 4, 8]
    assert pos.tolist() == [[0, 4], [5, 1], [2, 6], [7, 3]]


def test_moe_remote_routes_ignored():
    # tests/python/test_fused_moe.py:103-140
    tokens, experts, hidden, x, xs, gw, gs, dw, ds = _moe_case()
    ids = np.full((tokens, 1), 2, np.int32)
    w = np.ones((tokens, 1), np.float32)
    shared = np.full((tokens, hidden), 2.0, np.float16)
    out, pos, seqlens, _ = oracle.fused_moe(x, xs, gw, gs, dw, ds, ids, w, shared, rank_ep=0)
    np.testing.assert_array_equal(out, shared)
    assert (pos == -1).all() and (seqlens == 0).all()


def test_moe_nonuniform_scales_survive_routing():
    # tests/python/test_fused_moe.py:142-195
    tokens, experts, hidden, x, xs, gw, gs, dw, ds = _moe_case()
    scale = np.zeros_like(xs)
    for row, code in enumerate((0x30, 0x38, 0x30, 0x38)):
        for kb in range(8):
            scale[(kb // 4) * 512 + (row % 32) * 16 + (row // 32) * 4 + (kb % 4)] = code
    ids = np.array([[1], [0], [1], [0]], np.int32)
    w = np.ones((tokens, 1), np.float32)
    out, *_ = oracle.fused_moe(x, scale, gw, gs, dw, ds, ids, w)
    assert out[:, 0].astype(np.float32).tolist() == [8448.0, 33792.0, 8448.0, 33792.0]


def test_expert_major_handoff_matches_reroute():
    # tests/python/test_fused_moe.py:198-300
    rows, experts, hidden, inter = 5, 2, 128, 64
    rng = np.random.default_rng(7)
    L = oracle.lib()
    xb = np.array([L.oracle_f32_to_bf16(float(v)) for v in rng.normal(size=rows * hidden) * 0.25],
                  np.uint16).reshape(rows, hidden)
    packed, scales = oracle.quantize_expert(xb, [2, 3], [0, 2, 5], 128, True)
    gw = np.full((experts, 2 * inter, hidden // 2), 0x11, np.uint8)
    dw = np.full((experts, hidden, inter // 2), 0x11, np.uint8)
    gs = np.full((experts, 128 * oracle.scale_k_padded(hidden)), 0x38, np.uint8)
    ds = np.full((experts, 128 * oracle.scale_k_padded(inter)), 0x38, np.uint8)
    direct = oracle.expert_moe(packed, scales, gw, gs, dw, ds, [2, 3], [0, 2, 5], 128)
    base_in, base_scale = oracle.quantize_expert(xb, [rows], [0, rows], 128, True)
    ids = np.array([[0], [0], [1], [1], [1]], np.int32)
    out, *_ = oracle.fused_moe(base_in, base_scale.ravel(), gw, gs, dw, ds, ids,
                               np.ones((rows, 1), np.float32))
    np.testing.assert_array_equal(direct, out)


def test_workspace_size_mirrors_python_wrapper():
    # python/sm120_nvfp4/__init__.py:245-269
    def py(total_rows, hidden, inter, e, pad):
        total = 0
        for size in (total_rows * inter * 4, total_rows * inter // 2,
                     e * pad * oracle.scale_k_padded(inter), (e * 3 + 2) * 128, (e * 3 + 2) * 128,
                     e * 4, (e + 1) * 4):
            total = (total + 255) // 256 * 256 + size
        return (total + 255) // 256 * 256
    L = oracle.lib()
    for args in ((5, 128, 64, 2, 128), (32768, 7168, 2048, 256, 32768), (777, 512, 96, 7, 384)):
        assert L.oracle_expert_moe_workspace_size(*args) == py(*args)


def test_expf_accuracy_against_libm():
    L = oracle.lib()
    xs = np.concatenate([np.linspace(-104, 88.7, 20001), np.linspace(-12, 12, 20001)]).astype(np.float32)
    worst = 0.0
    for x in xs:
        got = L.oracle_expf(float(x))
        want = math.exp(float(x))
        want32 = np.float32(want)
        if want32 == 0 or not np.isfinite(want32):
            continue
        ulp = float(np.spacing(want32))
        worst = max(worst, abs(got - want) / ulp)
    assert worst < 2.0, worst
    assert L.oracle_silu(0.0) == 0.0 and abs(L.oracle_silu(1.0) - 0.7310585786) < 1e-6
    assert L.oracle_silu(-200.0) == 0.0 or L.oracle_silu(-200.0) == -0.0


def test_router_topk_against_numpy_restatement():
    # the router of the DeepSeek-shaped configuration, restated with numpy: same ids wherever the
    # float32 scores are distinct, weights equal to a few ulp
    from helpers import topk_routing
    rng = np.random.default_rng(12)
    logits = rng.standard_normal((64, 256), dtype=np.float32)
    ids, w = oracle.router_topk(logits, 8)
    scores = 1.0 / (1.0 + np.exp(-logits.astype(np.float64)))
    order = np.argsort(-scores, axis=1, kind="stable")[:, :8]
    np.testing.assert_array_equal(ids, order.astype(np.int32))
    picked = np.take_along_axis(scores, order, axis=1)
    np.testing.assert_allclose(w, picked / picked.sum(1, keepdims=True), rtol=2e-6)
    tie = np.zeros((1, 16), np.float32)
    ids, w = oracle.router_topk(tie, 4)
    assert ids.tolist() == [[0, 1, 2, 3]] and np.allclose(w, 0.25)
