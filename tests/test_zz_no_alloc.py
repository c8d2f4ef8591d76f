"""GPU test of b200_nvfp4_gemm_splitk_static: the split-K GEMM that keeps its FP32 partial sums
in a fixed array inside the library instead of a caller-provided workspace. Called through the C
ABI and compared with b200_nvfp4_gemm_splitk (same operands, caller workspace) and with the CPU
oracle, on calls issued back to back so that the second call meets the first one's leftovers in
the scratch array. The file name sorts last so that the test also runs after every other GPU test
has used the library."""
import numpy as np
import pytest
import torch

import oracle
from helpers import check_gemm_parity, randn_quantized

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from sm120_nvfp4_b200 import _lib
    lib = _lib.lib()  # must load: there is no fallback path
    lib.b200_nvfp4_set_tile_n(0)
    yield lib
    assert _lib.device_error() == 0, "a bounded wait inside a kernel timed out"


def _dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def _case(m, n, k, seed):
    a, sfa = randn_quantized(m, k, seed)
    b, sfb = randn_quantized(n, k, seed + 1)
    return a, sfa, b, sfb


def _run_both(L, m, n, k, split, seed):
    a, sfa, b, sfb = _case(m, n, k, seed)
    ref32, _ = oracle.gemm(a, b, sfa, sfb)
    da, db, dsfa, dsfb = _dev(a), _dev(b), _dev(sfa), _dev(sfb)
    stream = torch.cuda.current_stream().cuda_stream
    want = torch.empty((m, n), dtype=torch.float16, device="cuda")
    ws = torch.empty(split * m * n, dtype=torch.float32, device="cuda")
    assert L.b200_nvfp4_gemm_splitk(m, n, k, split, da.data_ptr(), db.data_ptr(), dsfa.data_ptr(), dsfb.data_ptr(),
                                    want.data_ptr(), ws.data_ptr(), ws.numel() * 4, stream) == 0
    got = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    assert L.b200_nvfp4_gemm_splitk_static(m, n, k, split, da.data_ptr(), db.data_ptr(), dsfa.data_ptr(),
                                           dsfb.data_ptr(), got.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    got, want = got.cpu().numpy(), want.cpu().numpy()
    check_gemm_parity(got, ref32)                       # the GEMM gate against the oracle
    check_gemm_parity(got, want.astype(np.float32))     # and against the workspace-taking entry point
    np.testing.assert_array_equal(got, want)            # same kernels, same order of additions


def test_static_scratch_splitk_matches_workspace_splitk_twice_in_a_row(L):
    # the larger problem first: the second, smaller call then finds stale partial sums in the scratch
    _run_both(L, 128, 1024, 2048, 4, seed=4100)
    _run_both(L, 256, 384, 1024, 2, seed=4200)
    # a k-split without work (more splits than 128-wide k-tiles allow is refused; equal is the edge)
    _run_both(L, 96, 136, 512, 4, seed=4300)
    # the same call twice: the result does not depend on what the previous call left behind
    _run_both(L, 128, 1024, 2048, 4, seed=4100)


def test_static_scratch_limit_is_enforced_without_launching(L):
    limit = L.b200_nvfp4_gemm_splitk_static_max_elements()
    assert limit == 4 << 20
    from sm120_nvfp4_b200 import _lib
    before = _lib.launch_count()
    m, n, k, split = 128, 8200, 512, 4                  # 4 * 128 * 8200 floats: just above the limit
    assert split * m * n > limit
    buf = torch.zeros(16, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    status = L.b200_nvfp4_gemm_splitk_static(m, n, k, split, buf.data_ptr(), buf.data_ptr(), buf.data_ptr(),
                                             buf.data_ptr(), buf.data_ptr(), stream)
    assert status == 3                                  # B200_NVFP4_INSUFFICIENT_WORKSPACE
    assert _lib.launch_count() == before
    # exactly at the limit is accepted (checked on shape arithmetic only: M*N*split == 4 Mi)
    assert 4 * 128 * 8192 == limit
    _run_both(L, 128, 8192, 512, 4, seed=4400)


def test_static_scratch_entry_leaves_device_memory_untouched(L):
    # "allocates nothing", measured: the driver's count of free device memory is the same before and
    # after calls of the entry point (first use of the kernels happened in the tests above; the
    # operands and the output are allocated before the first reading).
    m, n, k, split = 128, 1024, 2048, 4
    a, sfa, b, sfb = _case(m, n, k, 4500)
    da, db, dsfa, dsfb = _dev(a), _dev(b), _dev(sfa), _dev(sfb)
    out = torch.empty((m, n), dtype=torch.float16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        assert L.b200_nvfp4_gemm_splitk_static(m, n, k, split, da.data_ptr(), db.data_ptr(), dsfa.data_ptr(),
                                               dsfb.data_ptr(), out.data_ptr(), stream) == 0
        torch.cuda.synchronize()

    call()                                               # any first-use set-up happens here
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        call()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_static_scratch_rejects_sizes_that_would_overflow(L):
    # M and N near 2^31 with a large split: the element count does not fit 64 bits; the call must be
    # refused on arithmetic alone (no launch), and an over-large split_k is an invalid argument
    from sm120_nvfp4_b200 import _lib
    before = _lib.launch_count()
    buf = torch.zeros(16, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    huge = (1 << 31) - 8
    assert L.b200_nvfp4_gemm_splitk_static(huge, huge, 1 << 30, 1 << 22, p, p, p, p, p, None) == 3
    assert L.b200_nvfp4_gemm_splitk_static(128, 128, 256, 3, p, p, p, p, p, None) == 1      # > ceil(256 / 128) splits
    ws = torch.zeros(16, dtype=torch.float32, device="cuda")
    assert L.b200_nvfp4_gemm_splitk(huge, huge, 1 << 30, 1 << 22, p, p, p, p, p, ws.data_ptr(), 64, None) == 3
    assert _lib.launch_count() == before
