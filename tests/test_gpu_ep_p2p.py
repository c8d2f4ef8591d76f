"""Expert-parallel layer on two GPUs: the peer-memory transport (records and partial rows stored
straight into the peer's slots) against the all-to-all transport, same inputs, outputs bit for bit;
and the all-to-all transport against the per-rank composition of the CPU oracle. Needs two GPUs."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, result_dir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from sm120_nvfp4_b200.ep import ExpertParallelMoE
        from test_ep_gloo import _case, expected_ep_output
        # hidden = 256: two column blocks of 128 for the pipelined return path
        experts, hidden, inter, gw, gws, dw, dws, per_rank = _case(world, hidden=256)
        e_local = experts // world
        sl = slice(rank * e_local, (rank + 1) * e_local)
        weights = [torch.from_numpy(a[sl].copy()).to(dev) for a in (gw, gws, dw, dws)]
        xb, ids, w = per_rank[rank]
        x = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(dev)
        ids_t, w_t = torch.from_numpy(ids).to(dev), torch.from_numpy(w).to(dev)
        nccl = ExpertParallelMoE(*weights, experts)
        # both orderings of the hand-offs: per-rank ready words, and two full barriers per layer
        # and the down projection in column blocks with the return stores of a block on a second stream
        blocks = 2 if (weights[0].shape[2] * 2) % 256 == 0 else 1
        p2p = [ExpertParallelMoE(*weights, experts, transport="p2p", max_tokens=64, num_topk=ids.shape[1], handoff=h,
                                 return_blocks=b) for h, b in (("flags", 1), ("barrier", 1), ("flags", blocks))]
        ok = True
        for step in range(3):    # repeated calls reuse the slots
            a = nccl.forward(x, ids_t, w_t, out_bf16=False)
            for layer in p2p:
                b = layer.forward(x, ids_t, w_t, out_bf16=False)
                torch.cuda.synchronize()
                ok = ok and torch.equal(a, b)
        want = expected_ep_output(xb, ids, w, gw, gws, dw, dws, world)
        got = a.cpu().numpy().astype(np.float32)
        ref = want.astype(np.float32)
        frob = np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30)
        ok = ok and frob < 2e-2
        from sm120_nvfp4_b200 import _lib
        ok = ok and _lib.device_error() == 0
        Path(result_dir, f"rank{rank}.txt").write_text("ok" if ok else f"mismatch frob={frob}")
    finally:
        dist.destroy_process_group()


def test_p2p_transport_matches_all_to_all_on_two_gpus(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import torch.multiprocessing as mp
    world = 2
    port = 29700 + os.getpid() % 200
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"
