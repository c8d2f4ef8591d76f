"""Expert-parallel driver on two CPU ranks (gloo): the host logic - routing order, split
sizes, expert-major maps, the two exchanges, the combine - with the CPU oracle standing in
for the CUDA kernels, against the single-process oracle MoE. Bit-exact."""
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


class OracleBackend:
    """Checker backend: same interface as sm120_nvfp4_b200.ep.CudaBackend, numpy + oracle."""

    def route(self, topk_ids, num_experts):
        ids = topk_ids.numpy().reshape(-1)
        order = np.argsort(ids, kind="stable")
        pos = np.empty_like(ids)
        pos[order] = np.arange(ids.size, dtype=ids.dtype)
        seqlens = np.bincount(ids, minlength=num_experts).astype(np.int32)
        cu = np.concatenate([[0], np.cumsum(seqlens)]).astype(np.int32)
        return torch.from_numpy(pos.reshape(topk_ids.shape)), torch.from_numpy(seqlens), torch.from_numpy(cu)

    def scatter_rows(self, src, pos, rows_out):
        out = torch.zeros((rows_out, src.shape[1]), dtype=src.dtype)
        p = pos.reshape(-1).long()
        tok = torch.arange(p.numel()) // pos.shape[1]
        out[p] = src[tok]
        return out

    def gather_rows(self, src, index, rows_out):
        return src[index.long()[:rows_out]].clone()

    def quantize_gather(self, rows, row_map, seqlens, cu_seqlens, m_pad):
        import oracle
        gathered = rows[row_map.long()]
        bits = gathered.view(torch.int16).numpy().view(np.uint16)
        if bits.shape[0] == 0:
            bits = np.zeros((1, rows.shape[1]), np.uint16)
        packed, scales = oracle.quantize_expert(bits, seqlens.numpy(), cu_seqlens.numpy(), m_pad,
                                                rows.dtype == torch.bfloat16)
        return torch.from_numpy(packed), torch.from_numpy(scales)

    def expert_moe(self, packed, scales, gw, gws, dw, dws, seqlens, cu_seqlens, rows, m_pad):
        import oracle
        out = oracle.expert_moe(packed.numpy(), scales.numpy(), gw.numpy(), gws.numpy(), dw.numpy(), dws.numpy(),
                                seqlens.numpy(), cu_seqlens.numpy(), m_pad)
        return torch.from_numpy(out.copy())

    def reduce(self, rows, pos, weights, out_bf16):
        import oracle
        assert not out_bf16
        return torch.from_numpy(oracle.reduce(rows.numpy(), pos.numpy(), weights.numpy()).copy())


def _case(world):
    import oracle
    from helpers import randn_quantized, topk_routing
    experts, hidden, inter, topk, tokens = 8, 128, 64, 3, 37
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
        tokens = xb.shape[0]
        in_pad = (tokens + 127) // 128 * 128
        xq, xs = oracle.quantize_expert(xb, [tokens], [0, tokens], in_pad, True)
        want, *_ = oracle.fused_moe(xq, xs.ravel(), gw, gws, dw, dws, ids, w)
        ok = np.array_equal(out.numpy(), want)
        Path(result_dir, f"rank{rank}.txt").write_text("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_expert_parallel_matches_single_process_oracle(tmp_path, world):
    port = 29600 + os.getpid() % 200
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"


def test_expert_major_maps():
    from sm120_nvfp4_b200.ep import expert_major_maps
    counts = torch.tensor([[2, 0, 1], [1, 3, 0]], dtype=torch.int64)   # [source, expert]
    seqlens, cu, row_map, inv_map = expert_major_maps(counts, 7)
    assert seqlens.tolist() == [3, 3, 1] and cu.tolist() == [0, 3, 6, 7]
    # receive buffer: src0 = [e0,e0,e2], src1 = [e0,e1,e1,e1]
    assert row_map.tolist() == [0, 1, 3, 4, 5, 6, 2]
    assert inv_map[row_map.long()].tolist() == list(range(7))
