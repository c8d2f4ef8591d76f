"""GPU tests of the expert-parallel hand-off kernels (destination ranks, wire-record pack /
unpack) and of the expert-parallel layer on one rank, through the C ABI, against the numpy /
oracle checker backend used by the CPU multi-rank test. Integer and byte outputs bit-exact;
the layer output within the GEMM gate."""
import numpy as np
import pytest
import torch

import oracle
from helpers import check_gemm_parity, randn_quantized, topk_routing
from test_ep_gloo import OracleBackend, expected_ep_output

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def backend():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from sm120_nvfp4_b200 import _lib
    from sm120_nvfp4_b200.ep import CudaBackend
    _lib.lib()
    yield CudaBackend()
    assert _lib.device_error() == 0


def _bf16_rows(tokens, hidden, seed):
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.standard_normal((tokens, hidden), dtype=np.float32)).to(torch.bfloat16)
    return x


@pytest.mark.parametrize("tokens,experts,topk,world,hidden", [(37, 8, 3, 2, 128), (1500, 64, 8, 8, 448),
                                                               (4096, 256, 8, 4, 7168)])
def test_pack_and_unpack_match_checker(backend, tokens, experts, topk, world, hidden):
    chk = OracleBackend()
    ids, w = topk_routing(tokens, experts, topk, 77)
    x = _bf16_rows(tokens, hidden, 5)
    ids_t, w_t = torch.from_numpy(ids), torch.from_numpy(w)
    per_rank = experts // world
    dest = backend.dest_ranks(ids_t.cuda(), per_rank, world)
    want_dest = chk.dest_ranks(ids_t, per_rank, world)
    assert torch.equal(dest.cpu(), want_dest)
    pos, counts, cu = backend.route(dest, world)
    want_pos, want_counts, want_cu = chk.route(want_dest, world)
    assert torch.equal(pos.cpu(), want_pos) and torch.equal(counts.cpu(), want_counts) and torch.equal(cu.cpu(), want_cu)
    sent = int(want_cu[-1])
    rec = backend.pack_rows(x.cuda(), ids_t.cuda(), w_t.cuda(), pos, tokens * world)
    want_rec = chk.pack_rows(x, ids_t, w_t, want_pos, tokens * world)
    body = hidden // 2 + hidden // 16 + 8 * topk
    assert torch.equal(rec[:sent, :body].cpu(), want_rec[:sent, :body])
    # the receiving side, fed with the sender's records as they are
    xq, xs, rid, rw = backend.unpack_rows(rec[:sent].contiguous(), hidden, topk)
    wq, ws, wid, ww = chk.unpack_rows(want_rec[:sent], hidden, topk)
    assert torch.equal(xq.cpu(), wq) and torch.equal(rid.cpu(), wid) and torch.equal(rw.cpu(), ww)
    # scale bytes of live rows (the padding rows of the region are not written)
    nkb = hidden // 16
    r = np.repeat(np.arange(sent, dtype=np.int32), nkb)
    kb = np.tile(np.arange(nkb, dtype=np.int32), sent)
    off = oracle.sf_offsets(r, kb, hidden)
    np.testing.assert_array_equal(xs.cpu().numpy()[off], ws.numpy()[off])


def test_layer_on_one_rank_matches_oracle(backend):
    from sm120_nvfp4_b200.ep import ExpertParallelMoE
    experts, hidden, inter, topk, tokens = 8, 256, 128, 3, 200
    gw = np.empty((experts, 2 * inter, hidden // 2), np.uint8)
    gws = np.empty((experts, oracle.scale_region_bytes(2 * inter, hidden)), np.uint8)
    dw = np.empty((experts, hidden, inter // 2), np.uint8)
    dws = np.empty((experts, oracle.scale_region_bytes(hidden, inter)), np.uint8)
    for e in range(experts):
        gw[e], gws[e] = randn_quantized(2 * inter, hidden, 10 + 2 * e, 0.5)
        dw[e], dws[e] = randn_quantized(hidden, inter, 11 + 2 * e, 0.5)
    x = _bf16_rows(tokens, hidden, 9)
    ids, w = topk_routing(tokens, experts, topk, 31)
    layer = ExpertParallelMoE(torch.from_numpy(gw).cuda(), torch.from_numpy(gws).cuda(), torch.from_numpy(dw).cuda(),
                              torch.from_numpy(dws).cuda(), experts, backend=backend)
    out = layer.forward(x.cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), out_bf16=False)
    torch.cuda.synchronize()
    xb = x.view(torch.int16).numpy().view(np.uint16)
    want = expected_ep_output(xb, ids, w, gw, gws, dw, dws, 1)
    check_gemm_parity(out.cpu().numpy(), want.astype(np.float32))


class _EmulatedPeers:
    """Slotted buffers of one emulated rank; the pointer tables address every emulated rank's buffers."""

    def __init__(self, rank, world, slot_rows, hidden, topk, rec, cnt, ret, flags):
        import ctypes
        arr = ctypes.c_void_p * world
        self.my_rank, self.world = rank, world
        self.slot_rows, self.hidden, self.topk = slot_rows, hidden, topk
        self.peer_rec = arr(*[t.data_ptr() for t in rec])
        self.peer_cnt = arr(*[t.data_ptr() for t in cnt])
        self.peer_ret = arr(*[t.data_ptr() for t in ret])
        self.peer_flag = arr(*[t.data_ptr() for t in flags])
        self.rec, self.cnt, self.ret, self.flags = rec[rank], cnt[rank], ret[rank], flags[rank]
        self.step = 0

    def barrier(self):
        pass

    def publish(self, which):
        from sm120_nvfp4_b200.ep import publish_ready
        publish_ready(self.peer_flag, self.my_rank, self.world, which, self.step, self.flags.device)

    def ready_ptr(self, which):
        from sm120_nvfp4_b200.ep import ready_slot
        return self.flags.data_ptr() + 4 * ready_slot(which, self.world)


@pytest.mark.parametrize("handoff,return_blocks", [("flags", 1), ("barrier", 1), ("flags", 2)])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_memory_hand_off_emulated_on_one_gpu(backend, world, handoff, return_blocks):
    # All ranks of the peer-memory transport in one process on one GPU: every emulated rank has its
    # own slotted buffers, the pointer tables address the other ranks' buffers on the same device, and
    # the three phases of the layer run rank after rank: every rank has published its ready word (or
    # would have passed the barrier) before a kernel of the next phase looks for it, so no launch ever
    # waits on a later one.
    # Checks the layer code and the slot addressing of dispatch / unpack / reduce-and-return for more
    # than two ranks against the oracle's per-rank composition, over two calls (slot reuse).
    from sm120_nvfp4_b200 import _lib
    from sm120_nvfp4_b200.ep import ExpertParallelMoE, FLAG_WORDS, record_bytes
    # return_blocks = 2: the down projection in two column blocks, the return stores of the first on a
    # second stream beside the second block's GEMM
    experts, hidden, inter, topk, tokens, slot = 2 * world, 128 * return_blocks, 64, 3, 29, 32
    e_local = experts // world
    gw = np.empty((experts, 2 * inter, hidden // 2), np.uint8)
    gws = np.empty((experts, oracle.scale_region_bytes(2 * inter, hidden)), np.uint8)
    dw = np.empty((experts, hidden, inter // 2), np.uint8)
    dws = np.empty((experts, oracle.scale_region_bytes(hidden, inter)), np.uint8)
    for e in range(experts):
        gw[e], gws[e] = randn_quantized(2 * inter, hidden, 10 + 2 * e, 0.5)
        dw[e], dws[e] = randn_quantized(hidden, inter, 11 + 2 * e, 0.5)
    rows = world * slot
    rec = [torch.zeros((rows, record_bytes(hidden, topk)), dtype=torch.uint8, device="cuda") for _ in range(world)]
    cnt = [torch.zeros(world, dtype=torch.int32, device="cuda") for _ in range(world)]
    ret = [torch.zeros((rows, hidden), dtype=torch.float16, device="cuda") for _ in range(world)]
    flags = [torch.zeros(FLAG_WORDS, dtype=torch.int32, device="cuda") for _ in range(world)]
    layers = []
    for r in range(world):
        sl = slice(r * e_local, (r + 1) * e_local)
        peers = _EmulatedPeers(r, world, slot, hidden, topk, rec, cnt, ret, flags)
        layers.append(ExpertParallelMoE(*(torch.from_numpy(a[sl].copy()).cuda() for a in (gw, gws, dw, dws)), experts,
                                        backend=backend, transport="p2p", emulate=(world, r, peers), handoff=handoff,
                                        barrier_limit_cycles=1 << 20, return_blocks=return_blocks))
    for call in range(2):
        inputs, ret_pos = [], []
        for r in range(world):                               # phase 1 on every rank, then the barrier
            x = _bf16_rows(tokens - call, hidden, 100 + r + 10 * call).cuda()
            ids, w = topk_routing(tokens - call, experts, topk, 200 + r + 10 * call)
            ret_pos.append(layers[r].p2p_dispatch(x, torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()))
            inputs.append((x, ids, w))
        for r in range(world):                               # phase 2 on every rank, then the barrier
            layers[r].p2p_compute_and_return()
        for r in range(world):                               # phase 3
            out = layers[r].p2p_finish(ret_pos[r], out_bf16=False)
            torch.cuda.synchronize()
            x, ids, w = inputs[r]
            xb = x.cpu().view(torch.int16).numpy().view(np.uint16)
            want = expected_ep_output(xb, ids, w, gw, gws, dw, dws, world).astype(np.float32)
            got = out.cpu().numpy().astype(np.float32)
            frob = np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)
            assert frob < 1e-3, (call, r, frob)
            # the BF16 form of the final sum: the same FP32 sums, rounded to 8 significant bits
            out_b = layers[r].p2p_finish(ret_pos[r], out_bf16=True)
            torch.cuda.synchronize()
            assert out_b.dtype == torch.bfloat16
            diff = (out_b.float() - out.float()).abs()
            assert bool((diff <= out.float().abs() * 2.0 ** -8 + 2.0 ** -20).all())
    assert _lib.device_error() == 0                          # no wait ran out


def test_ready_word_that_never_arrives_is_reported_and_its_rows_are_left_out(backend):
    # The ready words of the peer-memory hand-off with a source that never publishes: two ranks'
    # slots on one GPU, only rank 0's "records delivered" word is set. The unpack kernel's wait for
    # rank 1 gives up after its limit (about half a millisecond), marks rank 1's rows empty, leaves
    # code 10 | 1 << 8 in the device error word and returns; rank 0's rows are unpacked. The final sum
    # reports a missing "partial rows delivered" word the same way (code 11) and still returns.
    from sm120_nvfp4_b200 import _lib
    from sm120_nvfp4_b200.ep import record_bytes
    from sm120_nvfp4_b200.ops import scale_k_padded
    L = _lib.lib()
    world, slot, hidden, topk = 2, 4, 128, 2
    rows = world * slot
    rb = record_bytes(hidden, topk)
    g = torch.Generator().manual_seed(5)
    rec = torch.randint(0, 256, (rows, rb), dtype=torch.uint8, generator=g)
    rec[:, hidden // 2 + hidden // 16:hidden // 2 + hidden // 16 + 4 * topk] = torch.tensor(
        [3, 0, 0, 0, 1, 0, 0, 0], dtype=torch.uint8)        # ids (3, 1) in every record
    rec = rec.cuda()
    cnt = torch.tensor([3, 2], dtype=torch.int32, device="cuda")
    ready = torch.tensor([7, 6], dtype=torch.int32, device="cuda")       # epoch 7: rank 1 is one step behind
    xq = torch.zeros((rows, hidden // 2), dtype=torch.uint8, device="cuda")
    xs = torch.zeros(128 * scale_k_padded(hidden), dtype=torch.uint8, device="cuda")
    ids = torch.zeros((rows, topk), dtype=torch.int32, device="cuda")
    wts = torch.ones((rows, topk), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert L.b200_nvfp4_ep_unpack_slots_ready(xq.data_ptr(), xs.data_ptr(), ids.data_ptr(), wts.data_ptr(),
                                              rec.data_ptr(), cnt.data_ptr(), world, slot, hidden, topk,
                                              ready.data_ptr(), 7, 1 << 20, stream) == _lib.STATUS_SUCCESS
    torch.cuda.synchronize()
    assert _lib.device_error() == (10 | (1 << 8))
    assert _lib.device_error() == 0
    assert ids.cpu().tolist() == [[3, 1]] * 3 + [[-1, -1]] * 5          # rank 0: 3 rows; rank 1: none taken
    assert torch.equal(xq[:3].cpu(), rec[:3, :hidden // 2].cpu())
    assert not wts[3:].any()
    ready[1] = 7                                                         # rank 1 publishes: everything is taken
    assert L.b200_nvfp4_ep_unpack_slots_ready(xq.data_ptr(), xs.data_ptr(), ids.data_ptr(), wts.data_ptr(),
                                              rec.data_ptr(), cnt.data_ptr(), world, slot, hidden, topk,
                                              ready.data_ptr(), 7, 1 << 20, stream) == _lib.STATUS_SUCCESS
    torch.cuda.synchronize()
    assert _lib.device_error() == 0
    assert ids.cpu().tolist() == [[3, 1]] * 3 + [[-1, -1]] + [[3, 1]] * 2 + [[-1, -1]] * 2
    # the final sum: partial rows of rank 1 not announced
    ret = torch.ones((rows, hidden), dtype=torch.float16, device="cuda")
    ret_pos = torch.tensor([[0, 4], [1, -1]], dtype=torch.int32, device="cuda")
    out = torch.zeros((2, hidden), dtype=torch.float16, device="cuda")
    ready[1] = 6
    assert L.b200_nvfp4_ep_sum_p2p(out.data_ptr(), ret.data_ptr(), ret_pos.data_ptr(), 2, hidden, world, 0,
                                   ready.data_ptr(), 7, 1 << 20, stream) == _lib.STATUS_SUCCESS
    torch.cuda.synchronize()
    assert _lib.device_error() == (11 | (1 << 8))
    ready[1] = 7
    assert L.b200_nvfp4_ep_sum_p2p(out.data_ptr(), ret.data_ptr(), ret_pos.data_ptr(), 2, hidden, world, 0,
                                   ready.data_ptr(), 7, 1 << 20, stream) == _lib.STATUS_SUCCESS
    torch.cuda.synchronize()
    assert _lib.device_error() == 0
    assert out.cpu().tolist() == [[2.0] * hidden, [1.0] * hidden]
    # the publishing half: epoch into word slot + my_rank of every peer, nobody waited for
    import ctypes
    words = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(world)]
    table = (ctypes.c_void_p * world)(*[w_.data_ptr() for w_ in words])
    assert L.b200_nvfp4_ep_publish_p2p(table, 1, world, 4, 9, stream) == _lib.STATUS_SUCCESS
    torch.cuda.synchronize()
    assert all(w_.tolist() == [0, 0, 0, 0, 0, 9, 0, 0] for w_ in words)
    assert L.b200_nvfp4_ep_publish_p2p(table, 2, world, 4, 9, stream) == _lib.STATUS_INVALID_ARGUMENT


def test_barrier_wait_runs_out_and_reports_the_late_rank(backend):
    # The cross-GPU barrier of the peer-memory transport with a peer that never arrives: rank 0 of a
    # two-rank flag set on one GPU, rank 1's flag is simply never written. The wait gives up after
    # its limit (about half a millisecond here), the launch returns, the device error word names the
    # late rank, reading it clears it, and once the flag is there the same barrier passes.
    import ctypes
    from sm120_nvfp4_b200 import _lib
    L = _lib.lib()
    world = 2
    flags = [torch.zeros(world, dtype=torch.int32, device="cuda") for _ in range(world)]
    table = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
    stream = torch.cuda.current_stream().cuda_stream
    assert L.b200_nvfp4_ep_barrier_p2p(table, 0, world, 1, 1 << 20, stream) == _lib.STATUS_SUCCESS
    torch.cuda.synchronize()
    assert _lib.device_error() == (9 | (1 << 8))        # code 9, waiting for rank 1
    assert _lib.device_error() == 0                      # read-and-clear
    assert flags[0].tolist() == [1, 0] and flags[1].tolist() == [1, 0]   # rank 0 published its epoch
    flags[0][1] = 1                                      # "rank 1 arrived"
    assert L.b200_nvfp4_ep_barrier_p2p(table, 0, world, 1, 1 << 20, stream) == _lib.STATUS_SUCCESS
    torch.cuda.synchronize()
    assert _lib.device_error() == 0
    # argument checks: a rank outside the world, a null table entry
    assert L.b200_nvfp4_ep_barrier_p2p(table, 2, world, 1, 0, stream) == _lib.STATUS_INVALID_ARGUMENT
    bad = (ctypes.c_void_p * world)(flags[0].data_ptr(), None)
    assert L.b200_nvfp4_ep_barrier_p2p(bad, 0, world, 1, 0, stream) == _lib.STATUS_INVALID_ARGUMENT
