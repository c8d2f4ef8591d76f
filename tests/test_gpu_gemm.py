"""GPU parity tests of the NVFP4 GEMM (dense, batched, FP32, split-K) against the CPU oracle
and the committed golden vectors. All calls go through the C ABI (via the Python ops)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from helpers import check_gemm_parity, randn_quantized

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import sm120_nvfp4_b200 as pkg
    from sm120_nvfp4_b200 import _lib
    _lib.lib()  # must load: there is no fallback path
    yield pkg
    _lib.lib().b200_nvfp4_set_tile_n(0)
    assert _lib.device_error() == 0


def _dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def _no_device_error():
    from sm120_nvfp4_b200 import _lib
    assert _lib.device_error() == 0, "a bounded wait inside a kernel timed out"


def _ones_case(ops, fn, m, n, k):
    a = torch.full((m, k // 2), 0x22, dtype=torch.uint8, device="cuda")
    b = torch.full((n, k // 2), 0x22, dtype=torch.uint8, device="cuda")
    sfa = torch.full((ops.scale_a_elements(m, n, k),), 0x38, dtype=torch.uint8, device="cuda")
    sfb = torch.full((ops.scale_b_elements(m, n, k),), 0x38, dtype=torch.uint8, device="cuda")
    out = fn(a, b, sfa, sfb)
    torch.cuda.synchronize()
    assert out.dtype == torch.float16 and tuple(out.shape) == (m, n)
    got = out.float().cpu().numpy()
    assert (got == float(k)).all(), f"{fn.__name__} m={m} n={n} k={k}: {np.unique(got)[:8]}"


@pytest.mark.parametrize("tile_n", [0, 64, 128, 256, 512])
def test_all_ones_known_answer(ops, tile_n):
    # tests/python/test_gemm.py:39-68,102-134 (+ K tails and every tile width)
    from sm120_nvfp4_b200 import _lib
    _lib.lib().b200_nvfp4_set_tile_n(tile_n)
    for m, n, k in ((16, 128, 128), (64, 136, 128), (129, 136, 128), (128, 128, 64), (8, 8, 32),
                    (130, 264, 96), (16, 512, 1024), (300, 520, 2080)):
        _ones_case(ops, ops.cute_gemm, m, n, k)
        _ones_case(ops, ops.gemm, m, n, k)
        _ones_case(ops, ops.cutlass_gemm, m, n, k)
    _no_device_error()


def test_specialized_dispatch_matches_generic(ops):
    # tests/python/test_gemm.py:70-100: M=128 / 256, N=128, K=512 (more splits than k-stages)
    for m in (128, 256):
        _ones_case(ops, ops.gemm, m, 128, 512)
        _ones_case(ops, ops.cute_gemm, m, 128, 512)
    _no_device_error()


@pytest.mark.parametrize("tile_n", [0, 64, 128, 256, 512])
def test_dyadic_random_payloads_exact(ops, golden_dir, tile_n):
    # tests/python/test_gemm.py:17-37: exact equality with the dequantised matmul
    from sm120_nvfp4_b200 import _lib
    _lib.lib().b200_nvfp4_set_tile_n(tile_n)
    g = np.load(golden_dir / "dyadic_gemm.npz")
    n, k = 256, 512
    for m in (7, 128, 256):
        a, b = _dev(g[f"a_{m}"]), _dev(g[f"b_{m}"])
        sfa = torch.full((ops.scale_a_elements(m, n, k),), 0x18, dtype=torch.uint8, device="cuda")
        sfb = torch.full((ops.scale_b_elements(m, n, k),), 0x20, dtype=torch.uint8, device="cuda")
        for fn in (ops.gemm, ops.cute_gemm):
            got = fn(a, b, sfa, sfb).cpu().numpy()
            np.testing.assert_array_equal(got, g[f"expected_{m}"], err_msg=f"{fn.__name__} m={m}")
    _no_device_error()


def _random_case(m, n, k, seed):
    a, sfa = randn_quantized(m, k, seed)
    b, sfb = randn_quantized(n, k, seed + 1)
    return a, sfa, b, sfb


@pytest.mark.parametrize("tile_n", [0, 64, 128, 256, 512])
@pytest.mark.parametrize("shape", [(16, 256, 512), (200, 328, 1056), (77, 40, 96), (128, 512, 2048)])
def test_random_scales_vs_oracle(ops, shape, tile_n):
    # non-uniform per-block scales: exercises the scale layout end to end
    from sm120_nvfp4_b200 import _lib
    _lib.lib().b200_nvfp4_set_tile_n(tile_n)
    m, n, k = shape
    a, sfa, b, sfb = _random_case(m, n, k, 100 + m)
    ref32, _ = oracle.gemm(a, b, sfa, sfb)
    for fn in (ops.cute_gemm, ops.gemm):
        got = fn(_dev(a), _dev(b), _dev(sfa), _dev(sfb)).cpu().numpy()
        check_gemm_parity(got, ref32)
    _no_device_error()


def test_config1_full_vs_oracle(ops):
    # M=16, N=4096, K=8192: the reference's CPU-reference shape, compared in full
    m, n, k = 16, 4096, 8192
    a, sfa, b, sfb = _random_case(m, n, k, 0xB2000100)
    ref32, _ = oracle.gemm(a, b, sfa, sfb)
    got = ops.gemm(_dev(a), _dev(b), _dev(sfa), _dev(sfb)).cpu().numpy()
    frob, worst = check_gemm_parity(got, ref32)
    print(f"C1 frob={frob:.2e} gate={worst:.3f}")
    _no_device_error()


@pytest.mark.parametrize("m", [128, 256, 1024, 4096])
def test_config2_m_sweep_sampled(ops, m):
    # N=4096, K=8192; M=128/256 take the split-K paths. Oracle on sampled rows x columns.
    n, k = 4096, 8192
    a, sfa, b, sfb = _random_case(m, n, k, 0xB2000200 + m)
    rng = np.random.default_rng(m)
    rows = np.sort(rng.choice(m, size=min(m, 24), replace=False)).astype(np.int32)
    cols = np.sort(rng.choice(n, size=384, replace=False)).astype(np.int32)
    ref = oracle.gemm_sampled(a, b, sfa, sfb, rows, cols)
    out = ops.gemm(_dev(a), _dev(b), _dev(sfa), _dev(sfb))
    got = out.cpu().numpy()[np.ix_(rows, cols)]
    check_gemm_parity(got, ref)
    if m in (128, 256):  # dispatcher and generic kernel agree within the gate as well
        got2 = ops.cute_gemm(_dev(a), _dev(b), _dev(sfa), _dev(sfb)).cpu().numpy()[np.ix_(rows, cols)]
        check_gemm_parity(got2, ref)
    _no_device_error()


def test_square_8192_sampled_and_linearity(ops):
    # full-size property checks: sampled oracle comparison, and doubling every A scale
    # (adding 8 to the UE4M3 exponent field) doubles the result exactly
    m = n = k = 8192
    a, sfa, b, sfb = _random_case(m, n, k, 0xB2000300)
    rng = np.random.default_rng(8192)
    rows = np.sort(rng.choice(m, size=16, replace=False)).astype(np.int32)
    cols = np.sort(rng.choice(n, size=256, replace=False)).astype(np.int32)
    ref = oracle.gemm_sampled(a, b, sfa, sfb, rows, cols)
    da, db, dsfa, dsfb = _dev(a), _dev(b), _dev(sfa), _dev(sfb)
    out = ops.gemm(da, db, dsfa, dsfb)
    check_gemm_parity(out.cpu().numpy()[np.ix_(rows, cols)], ref)
    sfa2 = np.where((sfa >= 8) & (sfa < 0x70), sfa + 8, sfa).astype(np.uint8)
    doubled_everywhere = bool(((sfa == 0) | ((sfa >= 8) & (sfa < 0x70))).all())
    out2 = ops.gemm(da, db, _dev(sfa2), dsfb)
    if doubled_everywhere:
        sel = torch.isfinite(out2) & (out.abs() >= 2.0 ** -13)
        assert torch.equal(out2[sel], (out * 2)[sel])
    _no_device_error()


def test_fp32_and_batched_entry_points(ops):
    from sm120_nvfp4_b200 import _lib
    L = _lib.lib()
    groups, m, n, k = 3, 130, 264, 320
    As, Bs, SAs, SBs, refs = [], [], [], [], []
    for g in range(groups):
        a, sfa, b, sfb = _random_case(m, n, k, 500 + 10 * g)
        As.append(a); Bs.append(b); SAs.append(sfa); SBs.append(sfb)
        refs.append(oracle.gemm(a, b, sfa, sfb)[0])
    a, b = _dev(np.stack(As)), _dev(np.stack(Bs))
    sfa, sfb = _dev(np.stack(SAs)), _dev(np.stack(SBs))
    stream = torch.cuda.current_stream().cuda_stream
    for tile_n in (0, 64, 256, 512):
        L.b200_nvfp4_set_tile_n(tile_n)
        c16 = torch.full((groups, m, n), float("nan"), dtype=torch.float16, device="cuda")
        c32 = torch.full((groups, m, n), float("nan"), dtype=torch.float32, device="cuda")
        assert L.b200_nvfp4_gemm(groups, m, n, k, a.data_ptr(), b.data_ptr(), sfa.data_ptr(),
                                 sfb.data_ptr(), c16.data_ptr(), 0, stream) == 0
        assert L.b200_nvfp4_gemm(groups, m, n, k, a.data_ptr(), b.data_ptr(), sfa.data_ptr(),
                                 sfb.data_ptr(), c32.data_ptr(), 1, stream) == 0
        torch.cuda.synchronize()
        for g in range(groups):
            check_gemm_parity(c16[g].cpu().numpy(), refs[g])
            got32 = c32[g].cpu().numpy()
            rel = np.abs(got32 - refs[g]).max() / np.abs(refs[g]).max()
            assert rel < 1e-5, rel
    L.b200_nvfp4_set_tile_n(0)
    _no_device_error()


def test_splitk_entry_point_and_workspace_contract(ops):
    from sm120_nvfp4_b200 import _lib
    L = _lib.lib()
    m, n, k = 128, 384, 2048
    a, sfa, b, sfb = _random_case(m, n, k, 900)
    ref32, _ = oracle.gemm(a, b, sfa, sfb)
    da, db, dsfa, dsfb = _dev(a), _dev(b), _dev(sfa), _dev(sfb)
    out = torch.empty((m, n), dtype=torch.float16, device="cuda")
    ws_bytes = L.b200_nvfp4_gemm_workspace_bytes(m, n, k)
    assert ws_bytes == 4 * m * n * 4
    ws = torch.zeros(ws_bytes // 4, dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert L.b200_nvfp4_gemm_auto(m, n, k, da.data_ptr(), db.data_ptr(), dsfa.data_ptr(), dsfb.data_ptr(),
                                  out.data_ptr(), ws.data_ptr(), ws_bytes - 4, stream) == 3
    assert L.b200_nvfp4_gemm_auto(m, n, k, da.data_ptr(), db.data_ptr(), dsfa.data_ptr(), dsfb.data_ptr(),
                                  out.data_ptr(), ws.data_ptr(), ws_bytes, stream) == 0
    torch.cuda.synchronize()
    check_gemm_parity(out.cpu().numpy(), ref32)
    # the workspace-taking entry leaves the four FP32 partial slices in the workspace; its output is
    # their sum in split order, and the dispatcher (which reduces the same partial tiles on chip,
    # through the cluster's shared memory) gives the same bits
    out2 = torch.empty_like(out)
    assert L.b200_nvfp4_gemm_splitk(m, n, k, 4, da.data_ptr(), db.data_ptr(), dsfa.data_ptr(), dsfb.data_ptr(),
                                    out2.data_ptr(), ws.data_ptr(), ws_bytes, stream) == 0
    torch.cuda.synchronize()
    partial = ws.view(4, m, n).cpu().numpy()
    np.testing.assert_array_equal(oracle.splitk_reduce(partial), out2.cpu().numpy())
    np.testing.assert_array_equal(out.cpu().numpy(), out2.cpu().numpy())
    _no_device_error()


@pytest.mark.parametrize("tile_n", [0, 64, 128])
@pytest.mark.parametrize("m,n,k,split", [(128, 4096, 8192, 4), (256, 4096, 8192, 2), (16, 4096, 8192, 2), (100, 136, 1024, 4),
                                         (256, 264, 768, 2), (300, 520, 2080, 4), (64, 64, 256, 2)])
def test_cluster_splitk_matches_workspace_splitk_bit_for_bit(ops, m, n, k, split, tile_n):
    # split-K reduced through distributed shared memory against the workspace + reduce-kernel form:
    # same K ranges, same order of FP32 additions, so the FP16 results are identical; ragged rows and
    # columns, several tiles per cluster (persistent loop, slot hand-back), a split without work
    from sm120_nvfp4_b200 import _lib
    L = _lib.lib()
    L.b200_nvfp4_set_tile_n(tile_n)
    a, sfa, b, sfb = _random_case(m, n, k, 1300 + m + split)
    da, db, dsfa, dsfb = _dev(a), _dev(b), _dev(sfa), _dev(sfb)
    stream = torch.cuda.current_stream().cuda_stream
    want = torch.empty((m, n), dtype=torch.float16, device="cuda")
    ws = torch.empty(split * m * n, dtype=torch.float32, device="cuda")
    assert L.b200_nvfp4_gemm_splitk(m, n, k, split, da.data_ptr(), db.data_ptr(), dsfa.data_ptr(), dsfb.data_ptr(),
                                    want.data_ptr(), ws.data_ptr(), ws.numel() * 4, stream) == 0
    for rep in range(2):
        got = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        assert L.b200_nvfp4_gemm_splitk_cluster(m, n, k, split, da.data_ptr(), db.data_ptr(), dsfa.data_ptr(),
                                                dsfb.data_ptr(), got.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        np.testing.assert_array_equal(got.cpu().numpy(), want.cpu().numpy())
    L.b200_nvfp4_set_tile_n(0)
    assert L.b200_nvfp4_gemm_splitk_cluster(m, n, k, 3, da.data_ptr(), db.data_ptr(), dsfa.data_ptr(), dsfb.data_ptr(),
                                            got.data_ptr(), stream) == _lib.STATUS_INVALID_ARGUMENT
    _no_device_error()


@pytest.mark.parametrize("m,n,k,block_rows,block_cols", [(300, 520, 1024, 128, 256), (1100, 4200, 1024, 0, 0),
                                                         (1000, 264, 512, 256, 128)])
def test_host_memory_gemm_matches_oracle(ops, m, n, k, block_rows, block_cols):
    # Operands and result in page-locked host memory, chunked copies overlapped with the blocks'
    # GEMMs. Ragged last chunks in both directions; the result must satisfy the GEMM gate against
    # the oracle and, over two calls on the same scratch, stay identical.
    a, sfa = randn_quantized(m, k, 501)
    b, sfb = randn_quantized(n, k, 502)
    host = [torch.from_numpy(np.ascontiguousarray(x)).pin_memory() for x in (a, b, sfa, sfb)]
    runner = ops.HostGemm(m, n, k, block_rows=block_rows, block_cols=block_cols)
    out = torch.zeros((m, n), dtype=torch.float16).pin_memory()
    ret = runner.run(*host, out=out)
    torch.cuda.synchronize()
    assert ret.data_ptr() == out.data_ptr()
    first = out.clone()
    want, _ = oracle.gemm(a, b, sfa, sfb)
    check_gemm_parity(first.numpy(), want)
    out.zero_()
    runner.run(*host, out=out)
    torch.cuda.synchronize()
    assert torch.equal(out, first)
    _no_device_error()


@pytest.mark.parametrize("tile_n", [64, 512])
def test_a_wait_that_runs_out_is_reported_and_leaves_the_library_usable(ops, tile_n):
    # The bounded-wait path of the GEMM kernel, exercised without anything faulting: the test hook
    # shortens the wait limit to about a millisecond and makes the next launch leave out one
    # barrier arrival, so the first k-stage of CTA 0 never becomes ready. The launch must return,
    # the device error word must name a wait code and CTA 0, reading it must clear it, and the
    # following ordinary launch must be correct (tensor memory was freed, nothing is left armed).
    from sm120_nvfp4_b200 import _lib
    L = _lib.lib()
    L.b200_nvfp4_set_tile_n(tile_n)
    m, n, k = 256, 512, 1024
    a, sfa, b, sfb = _random_case(m, n, k, 777)
    da, db, dsfa, dsfb = _dev(a), _dev(b), _dev(sfa), _dev(sfb)
    assert L.b200_nvfp4_set_wait_limit(1 << 21, 1) == 0
    try:
        ops.cute_gemm(da, db, dsfa, dsfb)
        torch.cuda.synchronize()
    finally:
        assert L.b200_nvfp4_set_wait_limit(0, 0) == 0
    err = _lib.device_error()
    assert err != 0 and (err >> 8) <= 1 and (err & 255) in (1, 2, 3, 4, 5), err    # CTA 0 (or its pair partner)
    assert _lib.device_error() == 0
    got = ops.cute_gemm(da, db, dsfa, dsfb).cpu().numpy()
    ref32, _ = oracle.gemm(a, b, sfa, sfb)
    check_gemm_parity(got, ref32)
    _no_device_error()


def test_tile_rules_table_and_tuner(ops):
    # What the built-in rules launch for the configurations the reference quotes (tile in the low 16
    # bits of b200_nvfp4_last_launch_tile, K ranges reduced inside a cluster above), that a table
    # entry replaces that choice for exactly its problem without changing a bit of the result, and
    # that the tuner times every candidate and installs the fastest.
    from sm120_nvfp4_b200 import _lib
    L = _lib.lib()
    L.b200_nvfp4_set_tile_n(0)                          # an earlier test may have left its override
    ops.clear_tuned_tiles()

    def launched():
        v = L.b200_nvfp4_last_launch_tile()
        return v & 0xffff, v >> 16

    def operands(m, n, k, seed):
        g = torch.Generator(device="cuda").manual_seed(seed)
        a = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, device="cuda", generator=g)
        b = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda", generator=g)
        sfa = torch.randint(0x30, 0x3a, (ops.scale_a_elements(m, n, k),), dtype=torch.uint8, device="cuda", generator=g)
        sfb = torch.randint(0x30, 0x3a, (ops.scale_b_elements(m, n, k),), dtype=torch.uint8, device="cuda", generator=g)
        return a, b, sfa, sfb

    def run(m, n, k):
        return ops.cute_gemm(*operands(m, n, k, 71))

    base = run(16, 4096, 8192)
    assert launched() == (128, 4)                       # skinny: 128-column tiles, K over a cluster of 4
    run(1024, 4096, 8192)
    assert launched() == (512, 1)                       # a wave of pair tiles
    run(16, 4096, 1024)
    assert launched() == (64, 1)                        # too few k-stages to split: narrow tiles on 64 SMs
    # the dispatcher's M = 128 path keeps its split whatever the table says
    assert L.b200_nvfp4_tune_set(1, 128, 4096, 8192, 0, 0, 256) == 0
    ops.gemm(*operands(128, 4096, 8192, 73))
    assert launched() == (128, 4)
    # an entry for the M = 16 problem: the generic entry point follows it, other shapes do not
    assert L.b200_nvfp4_tune_set(1, 16, 4096, 8192, 0, 0, 256) == 0
    tuned = run(16, 4096, 8192)
    assert launched() == (256, 1)
    assert torch.equal(tuned, base)                     # the tile is not part of the arithmetic
    run(32, 4096, 8192)
    assert launched() == (128, 4) and ops.tuned_tile(32, 4096, 8192) == 0
    ops.clear_tuned_tiles()
    run(16, 4096, 8192)
    assert launched() == (128, 4)
    # the tuner: every candidate timed, the fastest installed and used
    res = ops.autotune_gemm(64, 1024, 512, iters=5)
    assert sorted(res["us"]) == [64, 128, 256, 512] and all(t > 0 for t in res["us"].values())
    assert res["best"] == min(res["us"], key=res["us"].get) == ops.tuned_tile(64, 1024, 512)
    run(64, 1024, 512)
    assert launched()[0] == res["best"]
    res_g = ops.autotune_grouped_gemm([100, 0, 300, 50], 512, 256, iters=5, candidates=(128, 512))
    assert sorted(res_g["us"]) == [128, 512]
    assert ops.tuned_tile(450, 512, 256, groups=4, grouped=True) == res_g["best"]
    ops.clear_tuned_tiles()
    _no_device_error()
