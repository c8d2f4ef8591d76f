"""Run-to-run determinism under a cold-cache stress: the same launch repeated, with a large fill
kernel in between every few launches so that the first tiles of every persistent worker start with
cold caches and skewed CTAs, must give bit-identical outputs (every reduction order in the kernels
is fixed). Catches synchronisation races that single-shot parity tests miss."""
import numpy as np
import pytest
import torch

from helpers import dirichlet_counts

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


def _repeat(fn, reps, junk):
    first = fn().clone()
    for i in range(reps):
        if i % 3 == 0:
            junk.fill_(i & 255)
        out = fn()
        if not torch.equal(out, first):
            d = out != first
            rows = d.any(1).nonzero().flatten()
            cols = d.any(0).nonzero().flatten()
            pytest.fail(f"repetition {i}: {int(d.sum())} elements differ, rows {int(rows[0])}..{int(rows[-1])}, "
                        f"columns {int(cols[0])}..{int(cols[-1])}")


@pytest.mark.parametrize("tile_n", [0, 128, 512])
def test_grouped_gemm_is_deterministic(ops, tile_n):
    from sm120_nvfp4_b200 import _lib
    _lib.lib().b200_nvfp4_set_tile_n(tile_n)
    groups, total, n, k = 8, 2048, 4096, 8192
    counts, cu = dirichlet_counts(total, groups, 0xB2000300)
    pad = max(128, (int(counts.max()) + 127) // 128 * 128)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randint(0, 256, (total, k // 2), dtype=torch.uint8, device="cuda", generator=g)
    w = torch.randint(0, 256, (groups, n, k // 2), dtype=torch.uint8, device="cuda", generator=g)
    xs = torch.randint(0x28, 0x40, (groups, pad * ops.scale_k_padded(k)), dtype=torch.uint8, device="cuda", generator=g)
    ws = torch.randint(0x28, 0x40, (groups, n * ops.scale_k_padded(k)), dtype=torch.uint8, device="cuda", generator=g)
    dc, dcu = torch.from_numpy(counts).cuda(), torch.from_numpy(cu).cuda()
    junk = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")
    _repeat(lambda: ops.grouped_gemm(x, w, dc, dcu, xs, ws), 120, junk)


@pytest.mark.parametrize("tile_n", [0, 256, 64])
def test_dense_gemm_is_deterministic(ops, tile_n):
    from sm120_nvfp4_b200 import _lib
    _lib.lib().b200_nvfp4_set_tile_n(tile_n)
    m, n, k = 2048, 4096, 8192
    g = torch.Generator(device="cuda").manual_seed(2)
    a = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, device="cuda", generator=g)
    b = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda", generator=g)
    sfa = torch.randint(0x28, 0x40, (ops.scale_a_elements(m, n, k),), dtype=torch.uint8, device="cuda", generator=g)
    sfb = torch.randint(0x28, 0x40, (ops.scale_b_elements(m, n, k),), dtype=torch.uint8, device="cuda", generator=g)
    junk = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")
    _repeat(lambda: ops.cute_gemm(a, b, sfa, sfb), 120, junk)


@pytest.mark.parametrize("tile_n", [0, 128, 256])
def test_many_ragged_groups_finish_without_a_timed_out_wait(ops, tile_n):
    # 32 groups of about a thousand rows each, none a multiple of the tile height: every group ends
    # in a ragged tile whose rows leave by predicated stores, which hold up the other warps' shared
    # memory and barrier traffic for microseconds. A scale-mover warp delayed that long used to miss
    # a phase of a slot's `landed` barrier (the slot was released by the other team alone) and wait
    # for a phase that needed its own release: one launch in three ended in a timed-out wait.
    from sm120_nvfp4_b200 import _lib
    _lib.lib().b200_nvfp4_set_tile_n(tile_n)
    groups, n, k = 32, 4096, 7168
    rng = np.random.default_rng(0xB2000301)
    counts = (1024 + rng.integers(-75, 76, groups)).astype(np.int32)
    counts += (counts % 256 == 0)
    cu = np.zeros(groups + 1, np.int32)
    cu[1:] = np.cumsum(counts)
    total = int(cu[-1])
    pad = (int(counts.max()) + 127) // 128 * 128
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randint(0, 256, (total, k // 2), dtype=torch.uint8, device="cuda", generator=g)
    w = torch.randint(0, 256, (groups, n, k // 2), dtype=torch.uint8, device="cuda", generator=g)
    xs = torch.randint(0x28, 0x40, (groups, pad * ops.scale_k_padded(k)), dtype=torch.uint8, device="cuda", generator=g)
    ws = torch.randint(0x28, 0x40, (groups, n * ops.scale_k_padded(k)), dtype=torch.uint8, device="cuda", generator=g)
    dc, dcu = torch.from_numpy(counts).cuda(), torch.from_numpy(cu).cuda()
    junk = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _repeat(lambda: ops.grouped_gemm(x, w, dc, dcu, xs, ws), 60, junk)
    assert _lib.device_error() == 0


def test_calls_replayed_from_a_cuda_graph_give_the_eager_bits(ops):
    # The library enqueues on the caller's stream and neither allocates nor synchronises, so a sequence
    # of calls can be captured into a CUDA graph and replayed: a skinny GEMM (cluster split-K), the
    # dispatcher's M = 128 path, the token quantiser and a whole fused-MoE layer (routing, both grouped
    # GEMMs, the reduce), captured once after an eager warm-up, replayed - also on new inputs in the
    # same buffers - against the eager results bit for bit.
    from helpers import topk_routing
    g = torch.Generator(device="cuda").manual_seed(9)

    def rnd(shape, lo=0, hi=256):
        return torch.randint(lo, hi, shape, dtype=torch.uint8, device="cuda", generator=g)

    n, k = 1024, 2048
    a16, a128, b = rnd((16, k // 2)), rnd((128, k // 2)), rnd((n, k // 2))
    sfa16, sfa128 = rnd((ops.scale_a_elements(16, n, k),), 0x30, 0x3a), rnd((ops.scale_a_elements(128, n, k),), 0x30, 0x3a)
    sfb = rnd((ops.scale_b_elements(1, n, k),), 0x30, 0x3a)
    experts, hidden, inter, topk, tokens = 8, 256, 128, 2, 48
    gw, dw = rnd((experts, 2 * inter, hidden // 2)), rnd((experts, hidden, inter // 2))
    gws = rnd((experts, ops.scale_b_elements(1, 2 * inter, hidden)), 0x28, 0x30)
    dws = rnd((experts, ops.scale_b_elements(1, hidden, inter)), 0x28, 0x30)
    x = torch.randn((tokens, hidden), device="cuda", generator=g).to(torch.bfloat16)
    ids_np, w_np = topk_routing(tokens, experts, topk, 5)
    ids, wts = torch.from_numpy(ids_np).cuda(), torch.from_numpy(w_np).cuda()
    seq = torch.tensor([tokens], dtype=torch.int32, device="cuda")
    cu = torch.tensor([0, tokens], dtype=torch.int32, device="cuda")

    def work():
        xq, xs = ops.quantize_expert(x, seq, cu, scale_m_pad=128)
        return (ops.cute_gemm(a16, b, sfa16, sfb), ops.gemm(a128, b, sfa128, sfb),
                ops.fused_moe(xq, xs.flatten(), gw, gws, dw, dws, ids, wts))

    eager = [t.clone() for t in work()]                 # also the warm-up: one-time set-up happens here
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = work()
    for _ in range(3):
        for t in captured:
            t.fill_(0)
        graph.replay()
        torch.cuda.synchronize()
        for got, want in zip(captured, eager):
            assert torch.equal(got, want)
    # new inputs in the same buffers: the replay computes on what is there now
    a16.copy_(rnd((16, k // 2)))
    x.copy_(torch.randn((tokens, hidden), device="cuda", generator=g).to(torch.bfloat16))
    graph.replay()
    torch.cuda.synchronize()
    replayed = [t.clone() for t in captured]
    for got, want in zip(replayed, work()):
        assert torch.equal(got, want)
