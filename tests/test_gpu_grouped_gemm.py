"""GPU parity tests of the expert-grouped NVFP4 GEMM against the oracle and golden vectors."""
import numpy as np
import pytest
import torch

import oracle
from helpers import check_gemm_parity, dirichlet_counts, randn_quantized

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import sm120_nvfp4_b200 as pkg
    from sm120_nvfp4_b200 import _lib
    _lib.lib()
    yield pkg
    _lib.lib().b200_nvfp4_set_tile_n(0)
    assert _lib.device_error() == 0


def _dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


@pytest.mark.parametrize("tile_n", [0, 64, 128, 256, 512])
def test_empty_experts_tile_tails_and_changed_metadata(ops, golden_dir, tile_n):
    # tests/python/test_grouped_gemm.py:17-52: counts [0,1,127,129] then [129,0,1,127] on the
    # same buffers, NaN-prefilled output, exact equality
    from sm120_nvfp4_b200 import _lib
    _lib.lib().b200_nvfp4_set_tile_n(tile_n)
    g = np.load(golden_dir / "dyadic_gemm.npz")
    groups, rows, n, k, pad = 4, 257, 128, 128, 256
    x, weight = _dev(g["gx"]), _dev(g["gw"])
    codes = torch.from_numpy(g["gcodes"]).cuda()
    xs = codes[:, None].expand(-1, pad * ops.scale_k_padded(k)).contiguous()
    ws = codes.flip(0)[:, None].expand(-1, ops.scale_b_elements(1, n, k)).contiguous()
    lengths = torch.empty(groups, device="cuda", dtype=torch.int32)
    offsets = torch.empty(groups + 1, device="cuda", dtype=torch.int32)
    output = torch.empty((rows, n), device="cuda", dtype=torch.float16)
    for idx in range(2):
        counts = g[f"gcounts_{idx}"]
        prefix = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
        lengths.copy_(torch.from_numpy(counts))
        offsets.copy_(torch.from_numpy(prefix))
        output.fill_(float("nan"))
        actual = ops.grouped_gemm(x, weight, lengths, offsets, xs, ws, output=output)
        assert actual.data_ptr() == output.data_ptr()
        np.testing.assert_array_equal(actual.cpu().numpy(), g[f"gexpected_{idx}"])
    from sm120_nvfp4_b200 import _lib as l2
    assert l2.device_error() == 0


def test_uniform_scales(ops):
    # tests/python/test_grouped_gemm.py:54-85
    groups, total_m, n, k = 2, 5, 128, 128
    seqlens = torch.tensor([2, 3], dtype=torch.int32, device="cuda")
    cu = torch.tensor([0, 2, 5], dtype=torch.int32, device="cuda")
    x = torch.full((total_m, k // 2), 0x22, dtype=torch.uint8, device="cuda")
    w = torch.full((groups, n, k // 2), 0x22, dtype=torch.uint8, device="cuda")
    xs = torch.full((groups, 128 * 8), 0x38, dtype=torch.uint8, device="cuda")
    ws = torch.full((groups, 128 * 8), 0x38, dtype=torch.uint8, device="cuda")
    out = ops.grouped_gemm(x, w, seqlens, cu, xs, ws)
    assert tuple(out.shape) == (total_m, n) and out.dtype == torch.float16
    assert (out.float() == 128.0).all()


def test_rows_outside_groups_are_untouched_and_scratch_filled(ops):
    from sm120_nvfp4_b200 import _lib
    L = _lib.lib()
    groups, n, k, pad = 3, 136, 256, 128
    counts = np.array([5, 0, 100], np.int32)
    cu = np.array([0, 5, 5, 105], np.int32)
    rows = 140  # 35 trailing rows belong to no group
    x, _ = randn_quantized(rows, k, 11)
    xs = np.zeros((groups, pad * oracle.scale_k_padded(k)), np.uint8)
    w = np.zeros((groups, n, k // 2), np.uint8)
    ws = np.zeros((groups, oracle.scale_region_bytes(n, k)), np.uint8)
    for g in range(groups):
        w[g], ws[g] = randn_quantized(n, k, 20 + g)
        if counts[g]:
            _, xs_g = randn_quantized(int(counts[g]), k, 30 + g)  # scales only, for variety
            xs[g, :xs_g.size] = xs_g
    want = oracle.grouped_gemm(x, w, counts, cu, xs, ws, pad)
    y = torch.full((rows, n), 7.0, dtype=torch.float16, device="cuda")
    tiles = torch.full((groups,), -1, dtype=torch.int32, device="cuda")
    cu_tiles = torch.full((groups + 1,), -1, dtype=torch.int32, device="cuda")
    dx, dw, dxs, dws = _dev(x), _dev(w), _dev(xs), _dev(ws)
    dc, dcu = _dev(counts), _dev(cu)
    st = L.b200_nvfp4_grouped_gemm(y.data_ptr(), dx.data_ptr(), dw.data_ptr(), dc.data_ptr(), dcu.data_ptr(),
                                   dxs.data_ptr(), dws.data_ptr(), None, tiles.data_ptr(), cu_tiles.data_ptr(),
                                   groups, rows, n, k, pad, 35, 1, None, torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    assert (got[105:] == np.float16(7.0)).all()
    # oracle scales for padded rows differ from what the GPU saw only on rows >= counts
    ref32 = np.zeros((105, n), np.float32)
    for g in range(groups):
        if counts[g]:
            ref32[cu[g]:cu[g + 1]] = oracle.gemm(x[cu[g]:cu[g + 1]], w[g], xs[g], ws[g])[0]
    check_gemm_parity(got[:105], ref32)
    assert (got[:105] == want[:105]).mean() > 0.99  # FP16 roundings of the exact sum
    assert tiles.cpu().tolist() == [1, 0, 1] and cu_tiles.cpu().tolist() == [0, 1, 1, 2]
    assert _lib.device_error() == 0


@pytest.mark.parametrize("with_alpha", [False, True])
def test_config3_dirichlet_groups(ops, with_alpha):
    # E=8, 2048 rows split by a seeded Dirichlet(0.5) multinomial, N=4096, K=8192,
    # per-expert global scales U(0.5, 2) through the group_alpha extension
    groups, total, n, k = 8, 2048, 4096, 8192
    counts, cu = dirichlet_counts(total, groups, 0xB2000300)
    pad = max(128, (int(counts.max()) + 127) // 128 * 128)
    x, _ = randn_quantized(total, k, 0xB2000301)
    skp = oracle.scale_k_padded(k)
    xs = np.zeros((groups, pad * skp), np.uint8)
    rng = np.random.default_rng(0xB2000302)
    w = np.empty((groups, n, k // 2), np.uint8)
    ws = np.empty((groups, oracle.scale_region_bytes(n, k)), np.uint8)
    for g in range(groups):
        w[g], ws[g] = randn_quantized(n, k, 0xB2000310 + g)
        if counts[g]:
            xg = rng.standard_normal((int(counts[g]), k), dtype=np.float32)
            pk, sc = oracle.quantize_rows(xg)
            x[cu[g]:cu[g + 1]] = pk
            xs[g, :sc.size] = sc
    alpha = rng.uniform(0.5, 2.0, groups).astype(np.float32) if with_alpha else None
    out = ops.grouped_gemm(_dev(x), _dev(w), _dev(counts), _dev(cu), _dev(xs), _dev(ws),
                           group_alpha=None if alpha is None else _dev(alpha))
    got = out.cpu().numpy()
    cols = np.sort(rng.choice(n, size=192, replace=False)).astype(np.int32)
    for g in range(groups):
        if counts[g] == 0:
            continue
        r = np.sort(rng.choice(int(counts[g]), size=min(int(counts[g]), 6), replace=False)).astype(np.int32)
        ref = oracle.gemm_sampled(x[cu[g]:cu[g + 1]], w[g], xs[g], ws[g], r, cols,
                                  alpha=1.0 if alpha is None else float(alpha[g]))
        check_gemm_parity(got[cu[g] + r][:, cols], ref)
    from sm120_nvfp4_b200 import _lib
    assert _lib.device_error() == 0


@pytest.mark.parametrize("tile_n", [0, 64, 128, 256, 512])
def test_column_windows_write_the_same_bits_as_the_full_call(ops, tile_n):
    # b200_nvfp4_grouped_gemm_columns: the product computed block of columns by block of columns
    # (windows of 256, 128 and a ragged last one of 264 of N = 648) against the full call - same
    # bits inside the window, nothing written outside it; argument checks of the window.
    from sm120_nvfp4_b200 import _lib
    L = _lib.lib()
    L.b200_nvfp4_set_tile_n(tile_n)
    groups, n, k, pad = 3, 648, 256, 384
    counts = np.array([131, 0, 300], np.int32)
    cu = np.array([0, 131, 131, 431], np.int32)
    rows = 440
    x, _ = randn_quantized(rows, k, 41)
    xs = np.zeros((groups, pad * oracle.scale_k_padded(k)), np.uint8)
    w = np.zeros((groups, n, k // 2), np.uint8)
    ws = np.zeros((groups, oracle.scale_region_bytes(n, k)), np.uint8)
    for g in range(groups):
        w[g], ws[g] = randn_quantized(n, k, 50 + g)
        if counts[g]:
            _, xs_g = randn_quantized(int(counts[g]), k, 60 + g)
            xs[g, :xs_g.size] = xs_g
    dx, dw, dxs, dws, dc, dcu = _dev(x), _dev(w), _dev(xs), _dev(ws), _dev(counts), _dev(cu)
    alpha = torch.tensor([0.5, 2.0, 1.25], dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    full = torch.full((rows, n), 7.0, dtype=torch.float16, device="cuda")
    assert L.b200_nvfp4_grouped_gemm(full.data_ptr(), dx.data_ptr(), dw.data_ptr(), dc.data_ptr(), dcu.data_ptr(),
                                     dxs.data_ptr(), dws.data_ptr(), None, None, None, groups, rows, n, k, pad, 150,
                                     1, alpha.data_ptr(), stream) == 0

    def window(y, start, count):
        return L.b200_nvfp4_grouped_gemm_columns(y.data_ptr(), dx.data_ptr(), dw.data_ptr(), dc.data_ptr(),
                                                 dcu.data_ptr(), dxs.data_ptr(), dws.data_ptr(), groups, rows, n, k,
                                                 pad, 150, alpha.data_ptr(), start, count, stream)

    parts = torch.full((rows, n), 7.0, dtype=torch.float16, device="cuda")
    for start, count in ((256, 128), (0, 256), (384, 264)):
        one = torch.full((rows, n), 7.0, dtype=torch.float16, device="cuda")
        assert window(one, start, count) == 0
        assert window(parts, start, count) == 0
        torch.cuda.synchronize()
        assert torch.equal(one[:, start:start + count], full[:, start:start + count])
        outside = torch.ones(n, dtype=torch.bool, device="cuda")
        outside[start:start + count] = False
        assert (one[:, outside] == 7.0).all()
    assert torch.equal(parts, full)
    bad = _lib.STATUS_INVALID_ARGUMENT
    assert window(parts, 64, 128) == bad          # start not a multiple of 128
    assert window(parts, 0, 200) == bad           # inner window not a multiple of 128
    assert window(parts, 640, 128) == bad         # past the last column
    assert window(parts, 0, 0) == bad
    assert _lib.device_error() == 0
