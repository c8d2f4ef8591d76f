"""Expert-parallel driver on two CPU ranks (gloo): the host logic - destination ranks, send
order, split sizes, the two exchanges, the combine - with the CPU oracle standing in for the
CUDA kernels, against a single-process composition of the oracle. Bit-exact."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def _linear_scales(swizzled, rows, hidden):
    """Scale bytes [rows, hidden/16] read out of one block-scaled region."""
    import oracle
    nkb = hidden // 16
    r = np.repeat(np.arange(rows, dtype=np.int32), nkb)
    kb = np.tile(np.arange(nkb, dtype=np.int32), rows)
    return swizzled.ravel()[oracle.sf_offsets(r, kb, hidden)].reshape(rows, nkb)


class OracleBackend:
    """Checker backend: same interface as sm120_nvfp4_b200.ep.CudaBackend, numpy + oracle."""

    def dest_ranks(self, topk_ids, experts_per_rank, world):
        ids = topk_ids.numpy()
        dest = np.full((ids.shape[0], world), -1, np.int32)
        for r in range(world):
            hit = ((ids // experts_per_rank) == r).any(axis=1)
            dest[hit, r] = r
        return torch.from_numpy(dest)

    def route(self, ids, num_groups):
        flat = ids.numpy().reshape(-1)
        live = np.flatnonzero(flat >= 0)
        order = live[np.argsort(flat[live], kind="stable")]
        pos = np.full(flat.shape, -1, np.int32)
        pos[order] = np.arange(order.size, dtype=np.int32)
        seqlens = np.bincount(flat[live], minlength=num_groups).astype(np.int32)
        cu = np.concatenate([[0], np.cumsum(seqlens)]).astype(np.int32)
        return torch.from_numpy(pos.reshape(ids.shape)), torch.from_numpy(seqlens), torch.from_numpy(cu)

    def pack_rows(self, x, topk_ids, topk_weights, send_pos, rows_out):
        import oracle
        from sm120_nvfp4_b200.ep import record_bytes
        t, hidden = x.shape
        k = topk_ids.shape[1]
        bits = x.view(torch.int16).numpy().view(np.uint16)
        in_pad = (t + 127) // 128 * 128
        xq, xs = oracle.quantize_expert(bits, [t], [0, t], in_pad, x.dtype == torch.bfloat16)
        lin = _linear_scales(xs, t, hidden)
        rec = np.zeros((rows_out, record_bytes(hidden, k)), np.uint8)
        body = np.concatenate([xq, lin, topk_ids.numpy().view(np.uint8).reshape(t, 4 * k),
                               topk_weights.numpy().view(np.uint8).reshape(t, 4 * k)], axis=1)
        pos = send_pos.numpy()
        for r in range(pos.shape[1]):
            live = pos[:, r] >= 0
            rec[pos[live, r], :body.shape[1]] = body[live]
        return torch.from_numpy(rec)

    def unpack_rows(self, records, hidden, topk):
        import oracle
        rec = records.numpy()
        rows = rec.shape[0]
        nkb = hidden // 16
        xq = rec[:, :hidden // 2].copy()
        lin = rec[:, hidden // 2:hidden // 2 + nkb]
        m_pad = max(128, (rows + 127) // 128 * 128)
        xs = np.zeros(m_pad * oracle.scale_k_padded(hidden), np.uint8)
        r = np.repeat(np.arange(rows, dtype=np.int32), nkb)
        kb = np.tile(np.arange(nkb, dtype=np.int32), rows)
        xs[oracle.sf_offsets(r, kb, hidden)] = lin.reshape(-1)
        o = hidden // 2 + nkb
        ids = rec[:, o:o + 4 * topk].copy().view(np.int32)
        wts = rec[:, o + 4 * topk:o + 8 * topk].copy().view(np.float32)
        return torch.from_numpy(xq), torch.from_numpy(xs), torch.from_numpy(ids), torch.from_numpy(wts)

    def local_moe(self, xq, xs, ids, wts, gw, gws, dw, dws, rank, num_experts_total):
        import oracle
        out, *_ = oracle.fused_moe(xq.numpy(), xs.numpy(), gw.numpy(), gws.numpy(), dw.numpy(), dws.numpy(),
                                   ids.numpy(), wts.numpy(), rank_ep=rank)
        return torch.from_numpy(out.copy())

    def reduce(self, rows, pos, weights, out_bf16):
        import oracle
        assert not out_bf16
        return torch.from_numpy(oracle.reduce(rows.numpy(), pos.numpy(), weights.numpy()).copy())


def expected_ep_output(xb, ids, w, gw, gws, dw, dws, world):
    """What the expert-parallel layer must return for one source rank's tokens: per expert rank the
    FP16 partial sum over that rank's experts (the fused MoE with rank_ep set), then the partial
    rows added in ascending rank order in FP32 and rounded once."""
    import oracle
    tokens = xb.shape[0]
    experts = gw.shape[0]
    e_local = experts // world
    in_pad = (tokens + 127) // 128 * 128
    xq, xs = oracle.quantize_expert(xb, [tokens], [0, tokens], in_pad, True)
    parts, pos = [], np.full((tokens, world), -1, np.int32)
    for r in range(world):
        sl = slice(r * e_local, (r + 1) * e_local)
        part, *_ = oracle.fused_moe(xq, xs.ravel(), gw[sl], gws[sl], dw[sl], dws[sl], ids, w, rank_ep=r)
        parts.append(part)
        hit = ((ids // e_local) == r).any(axis=1)
        pos[hit, r] = r * tokens + np.flatnonzero(hit)
    stacked = np.concatenate(parts, axis=0)
    return oracle.reduce(stacked, pos, np.ones((tokens, world), np.float32))


def _case(world, hidden=128):
    import oracle
    from helpers import randn_quantized, topk_routing
    experts, inter, topk, tokens = 8, 64, 3, 37
    rng = np.random.default_rng(3)
    L = oracle.lib()
    gw = np.empty((experts, 2 * inter, hidden // 2), np.uint8)
    gws = np.empty((experts, oracle.scale_region_bytes(2 * inter, hidden)), np.uint8)
    dw = np.empty((experts, hidden, inter // 2), np.uint8)
    dws = np.empty((experts, oracle.scale_region_bytes(hidden, inter)), np.uint8)
    for e in range(experts):
        gw[e], gws[e] = randn_quantized(2 * inter, hidden, 10 + 2 * e, 0.5)
        dw[e], dws[e] = randn_quantized(hidden, inter, 11 + 2 * e, 0.5)
    per_rank = []
    for r in range(world):
        xb = np.array([L.oracle_f32_to_bf16(float(v)) for v in rng.standard_normal(tokens * hidden)],
                      np.uint16).reshape(tokens, hidden)
        ids, w = topk_routing(tokens, experts, topk, 100 + r)
        per_rank.append((xb, ids, w))
    return experts, hidden, inter, gw, gws, dw, dws, per_rank


def _worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from sm120_nvfp4_b200.ep import ExpertParallelMoE
        experts, hidden, inter, gw, gws, dw, dws, per_rank = _case(world)
        e_local = experts // world
        sl = slice(rank * e_local, (rank + 1) * e_local)
        layer = ExpertParallelMoE(torch.from_numpy(gw[sl].copy()), torch.from_numpy(gws[sl].copy()),
                                  torch.from_numpy(dw[sl].copy()), torch.from_numpy(dws[sl].copy()), experts,
                                  backend=OracleBackend())
        xb, ids, w = per_rank[rank]
        x = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16)
        out = layer.forward(x, torch.from_numpy(ids), torch.from_numpy(w), out_bf16=False)
        want = expected_ep_output(xb, ids, w, gw, gws, dw, dws, world)
        single = expected_ep_output(xb, ids, w, gw, gws, dw, dws, 1)
        # bit-exact against the per-rank composition; against the single-rank layer only the FP16
        # rounding of the per-rank partial sums differs
        ok = np.array_equal(out.numpy(), want)
        dev = np.abs(out.numpy().astype(np.float32) - single.astype(np.float32)).max()
        ok = ok and dev <= 4e-3 * max(np.abs(single.astype(np.float32)).max(), 1e-6)
        Path(result_dir, f"rank{rank}.txt").write_text("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_expert_parallel_matches_single_process_oracle(tmp_path, world):
    port = 29600 + os.getpid() % 200
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"


def _leaving_worker(rank, world, port, result_dir):
    """Rank 1 runs one layer and leaves (between steps, nothing of its own in flight); rank 0's next
    layer must end with an error inside the process-group timeout, not wait for ever."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    outcome = "no error"
    try:
        from sm120_nvfp4_b200.ep import ExpertParallelMoE
        experts, hidden, inter, gw, gws, dw, dws, per_rank = _case(world)
        e_local = experts // world
        sl = slice(rank * e_local, (rank + 1) * e_local)
        layer = ExpertParallelMoE(torch.from_numpy(gw[sl].copy()), torch.from_numpy(gws[sl].copy()),
                                  torch.from_numpy(dw[sl].copy()), torch.from_numpy(dws[sl].copy()), experts,
                                  backend=OracleBackend())
        xb, ids, w = per_rank[rank]
        x = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16)
        layer.forward(x, torch.from_numpy(ids), torch.from_numpy(w), out_bf16=False)     # step 0: both ranks
        if rank == 1:
            outcome = "left"
        else:
            try:
                layer.forward(x, torch.from_numpy(ids), torch.from_numpy(w), out_bf16=False)   # step 1: alone
            except Exception as exc:      # the exchange reports the missing peer
                outcome = "raised " + type(exc).__name__
    finally:
        Path(result_dir, f"rank{rank}.txt").write_text(outcome)
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_a_rank_that_leaves_between_steps_ends_the_next_exchange_with_an_error(tmp_path):
    world = 2
    port = 29400 + os.getpid() % 200
    mp.spawn(_leaving_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert (tmp_path / "rank1.txt").read_text() == "left"
    assert (tmp_path / "rank0.txt").read_text().startswith("raised")


def test_layer_options_are_checked_on_the_host():
    # Constructor checks of the expert-parallel layer that need no device: transport, hand-off and
    # column-block arguments, the expert split, and the epoch arithmetic of the ready words.
    from sm120_nvfp4_b200.ep import BARRIER_WORDS, FLAG_WORDS, ExpertParallelMoE, ready_slot, wrap_epoch
    hidden, inter, experts = 256, 64, 2
    gw = torch.zeros((experts, 2 * inter, hidden // 2), dtype=torch.uint8)
    gws = torch.zeros((experts, 1), dtype=torch.uint8)
    dw = torch.zeros((experts, hidden, inter // 2), dtype=torch.uint8)
    dws = torch.zeros((experts, 1), dtype=torch.uint8)
    backend = OracleBackend()
    layer = ExpertParallelMoE(gw, gws, dw, dws, experts, backend=backend)
    assert layer.world == 1 and layer.return_blocks == 1 and layer.handoff == "flags"
    assert ExpertParallelMoE(gw, gws, dw, dws, experts, backend=backend, return_blocks=2).return_blocks == 2
    for bad in (dict(transport="rdma"), dict(handoff="events"), dict(return_blocks=3), dict(return_blocks=-1)):
        with pytest.raises(ValueError):
            ExpertParallelMoE(gw, gws, dw, dws, experts, backend=backend, **bad)
    with pytest.raises(ValueError):
        ExpertParallelMoE(gw, gws, dw, dws, experts + 1, backend=backend)       # experts do not split over the ranks
    with pytest.raises(ValueError):
        ExpertParallelMoE(gw, gws, dw, dws, experts, backend=backend, transport="p2p")   # needs max_tokens, num_topk
    # ready words: after the barrier's words, `world` per kind, inside the flag area up to 64 ranks
    assert ready_slot("dispatch", 8) == BARRIER_WORDS and ready_slot("return", 8) == BARRIER_WORDS + 8
    assert ready_slot("return", 64) + 64 <= FLAG_WORDS
    # epochs are compared as signed 32-bit differences, so the step counter may wrap
    assert wrap_epoch(5) == 5 and wrap_epoch(2 ** 31 - 1) == 2 ** 31 - 1
    assert wrap_epoch(2 ** 31) == -2 ** 31 and wrap_epoch(2 ** 32 + 3) == 3
