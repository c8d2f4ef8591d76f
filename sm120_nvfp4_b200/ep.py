"""Expert-parallel fused MoE over the GPUs of one node.

Rank r owns the contiguous expert interval [r*E/W, (r+1)*E/W) - the convention of the
reference's rank_ep / num_expert_local arguments (src/fused_moe/count_and_gather.cu:106-107).
The exchange pattern follows the reference's only multi-GPU code, the 2-GPU hand-off benchmark
benchmarks/integration/benchmark_deepep_handoff.py (:55-58 counts, :356-364 dispatch,
:435-448 combine): an all-to-all of counts, an all-to-all of token rows each way, with the
fused MoE as the compute between them. What differs from that script:

  * a token travels ONCE to each rank that owns at least one of its experts (not once per
    expert), already quantised to NVFP4 and with its expert ids and route weights in the same
    wire record (4096 bytes for H = 7168, top-8, against 8 x 14336 bytes of BF16 rows);
  * the receiving rank runs the whole routed pipeline (`fused_moe` with rank_ep set: local
    routing, both grouped GEMMs, SiLU * up + requantisation, route-weighted sum over the local
    experts) and returns ONE partial row per received token;
  * the source rank adds the partial rows of a token in ascending rank order in FP32.

Packing, unpacking, routing and the final sum are this library's CUDA kernels
(b200_nvfp4_ep_dest_ranks / _ep_pack_rows / _ep_unpack_rows, b200_nvfp4_moe_route / _reduce).
torch.distributed (NCCL over NVLink / NVSwitch, gloo on CPU) is the transport; the split sizes
of the row exchanges are read back to the host once per call, as in the reference script. All
kernels read and write local HBM only.

The compute steps go through a small backend object so that the host logic (splits, ordering,
the two exchanges) can be exercised on CPU ranks with a checker backend supplied by the tests;
the default backend calls the C ABI and needs a CUDA device.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import _lib
from .ops import scale_k_padded


def record_bytes(hidden: int, topk: int) -> int:
    """Bytes of one wire record: payload, k-block-ordered scales, ids, weights, 16-byte padded."""
    return (hidden // 2 + hidden // 16 + 8 * topk + 15) // 16 * 16


class CudaBackend:
    """The product path: every step is a call into the C ABI on torch's current stream."""

    def __init__(self):
        self.L = _lib.lib()

    @staticmethod
    def _stream(t: torch.Tensor) -> int:
        return torch.cuda.current_stream(t.device).cuda_stream

    def dest_ranks(self, topk_ids, experts_per_rank, world):
        t, k = topk_ids.shape
        dest = torch.empty((t, world), dtype=torch.int32, device=topk_ids.device)
        _lib.check(self.L.b200_nvfp4_ep_dest_ranks(topk_ids.data_ptr(), dest.data_ptr(), t, k, experts_per_rank,
                                                   world, self._stream(topk_ids)), "ep_dest_ranks")
        return dest

    def route(self, ids, num_groups):
        t, k = ids.shape
        dev = ids.device
        pos = torch.empty((t, k), dtype=torch.int32, device=dev)
        seqlens = torch.empty(num_groups, dtype=torch.int32, device=dev)
        cu = torch.empty(num_groups + 1, dtype=torch.int32, device=dev)
        _lib.check(self.L.b200_nvfp4_moe_route(ids.data_ptr(), pos.data_ptr(), seqlens.data_ptr(),
                                               cu.data_ptr(), t, k, num_groups, 0, self._stream(ids)),
                   "moe_route")
        return pos, seqlens, cu

    def pack_rows(self, x, topk_ids, topk_weights, send_pos, rows_out):
        t, hidden = x.shape
        k, world = topk_ids.shape[1], send_pos.shape[1]
        rb = self.L.b200_nvfp4_ep_record_bytes(hidden, k)
        rec = torch.empty((rows_out, rb), dtype=torch.uint8, device=x.device)
        _lib.check(self.L.b200_nvfp4_ep_pack_rows(rec.data_ptr(), x.data_ptr(), topk_ids.data_ptr(),
                                                  topk_weights.data_ptr(), send_pos.data_ptr(), t, hidden, k, world,
                                                  int(x.dtype == torch.bfloat16), self._stream(x)), "ep_pack_rows")
        return rec

    def unpack_rows(self, records, hidden, topk):
        rows = records.shape[0]
        dev = records.device
        m_pad = max(128, (rows + 127) // 128 * 128)
        xq = torch.empty((rows, hidden // 2), dtype=torch.uint8, device=dev)
        xs = torch.empty(m_pad * scale_k_padded(hidden), dtype=torch.uint8, device=dev)
        ids = torch.empty((rows, topk), dtype=torch.int32, device=dev)
        wts = torch.empty((rows, topk), dtype=torch.float32, device=dev)
        _lib.check(self.L.b200_nvfp4_ep_unpack_rows(xq.data_ptr(), xs.data_ptr(), ids.data_ptr(), wts.data_ptr(),
                                                    records.data_ptr(), rows, hidden, topk, self._stream(records)),
                   "ep_unpack_rows")
        return xq, xs, ids, wts

    def local_moe(self, xq, xs, ids, wts, gate_up_w, gate_up_ws, down_w, down_ws, rank, num_experts_total):
        from . import ops
        return ops.fused_moe(xq, xs, gate_up_w, gate_up_ws, down_w, down_ws, ids, wts, ep_rank=rank,
                             num_experts=num_experts_total)

    def reduce(self, rows, pos, weights, out_bf16):
        t, k = pos.shape
        hidden = rows.shape[1]
        out = torch.empty((t, hidden), dtype=torch.bfloat16 if out_bf16 else torch.float16, device=rows.device)
        _lib.check(self.L.b200_nvfp4_moe_reduce(out.data_ptr(), rows.data_ptr(), pos.data_ptr(), weights.data_ptr(),
                                                None, t, hidden, k, int(out_bf16), self._stream(rows)), "moe_reduce")
        return out


class ExpertParallelMoE:
    """One MoE layer whose experts are sharded over the ranks of `group`.

    gate_up_weight [E_local, 2I, H/2], down_weight [E_local, H, I/2] (packed E2M1) and their
    scale regions are this rank's experts. forward() takes this rank's tokens (BF16 or FP16
    [T, H]), their top-k expert ids over all E experts and the route weights, and returns
    [T, H] (BF16 by default).
    """

    def __init__(self, gate_up_weight, gate_up_weight_scale, down_weight, down_weight_scale, num_experts_total: int,
                 group: Optional[dist.ProcessGroup] = None, backend=None):
        self.gw, self.gws, self.dw, self.dws = gate_up_weight, gate_up_weight_scale, down_weight, down_weight_scale
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.num_experts_total = int(num_experts_total)
        self.e_local = gate_up_weight.shape[0]
        if self.e_local * self.world != self.num_experts_total:
            raise ValueError("num_experts_total must equal world_size * local experts")
        self.backend = backend if backend is not None else CudaBackend()
        self.last_bytes = {"dispatch": 0, "combine": 0}
        self._ones = None

    def _all_to_all_rows(self, send, send_splits, recv_splits):
        recv = torch.empty((sum(recv_splits), send.shape[1]), dtype=send.dtype, device=send.device)
        if self.world == 1:
            recv.copy_(send)
        else:
            dist.all_to_all_single(recv, send, recv_splits, send_splits, group=self.group)
        return recv

    @torch.no_grad()
    def forward(self, x, topk_ids, topk_weights, out_bf16: bool = True):
        w, be = self.world, self.backend
        t, hidden = x.shape
        k = topk_ids.shape[1]
        # 1. which ranks does each token visit, and at which row of the rank-major send buffer
        dest = be.dest_ranks(topk_ids, self.e_local, w)
        send_pos, send_counts, _ = be.route(dest, w)
        # 2. row counts to every destination; quantise + pack while the host waits for them
        recv_counts = torch.empty_like(send_counts)
        if w == 1:
            recv_counts.copy_(send_counts)
        else:
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        records = be.pack_rows(x, topk_ids, topk_weights, send_pos, t * w)
        host = torch.cat((send_counts, recv_counts)).cpu()          # the one host read-back
        send_splits, recv_splits = host[:w].tolist(), host[w:].tolist()
        sent = int(sum(send_splits))
        # 3. dispatch
        got = self._all_to_all_rows(records[:sent], send_splits, recv_splits)
        self.last_bytes["dispatch"] = (sent - send_splits[self.rank]) * records.shape[1]
        rows = got.shape[0]
        # 4. the routed pipeline over this rank's experts: one partial row per received token
        if rows:
            xq, xs, ids, wts = be.unpack_rows(got, hidden, k)
            part = be.local_moe(xq, xs, ids, wts, self.gw, self.gws, self.dw, self.dws, self.rank,
                                self.num_experts_total)
        else:
            part = torch.empty((0, hidden), dtype=torch.float16, device=x.device)
        # 5. combine: partial rows back to their sources, summed there in ascending rank order
        ret = self._all_to_all_rows(part, recv_splits, send_splits)
        self.last_bytes["combine"] = (rows - recv_splits[self.rank]) * hidden * 2
        if self._ones is None or self._ones.shape != (t, w) or self._ones.device != x.device:
            self._ones = torch.ones((t, w), dtype=torch.float32, device=x.device)
        return be.reduce(ret, send_pos, self._ones, out_bf16)
