"""Expert-parallel fused MoE over the GPUs of one node.

Rank r owns the contiguous expert interval [r*E/W, (r+1)*E/W) - the convention of the
reference's rank_ep / num_expert_local arguments (src/fused_moe/count_and_gather.cu:106-107).
The exchange pattern follows the reference's only multi-GPU code, the 2-GPU hand-off benchmark
benchmarks/integration/benchmark_deepep_handoff.py (:55-58 counts, :356-364 dispatch,
:435-448 combine): one all-to-all of per-expert counts, one all-to-all of token rows each
way, with `expert_moe` as the compute between them. What differs from that script:

  * routing, the row scatter / gather and the weighted combine run in this library's CUDA
    kernels (b200_nvfp4_moe_route / _scatter_rows / _gather_rows / _reduce);
  * received rows are quantised to NVFP4 and permuted to expert-major order in one kernel
    (b200_nvfp4_moe_quantize_expert_gather) instead of an index_select plus a quantise;
  * route weights are applied once, in FP32, by the combine kernel on the source rank (the
    script multiplies on the expert rank in BF16 and index_adds in FP32).

torch.distributed (NCCL over NVLink / NVSwitch, gloo on CPU) is the transport; the split sizes
of the row exchanges are read back to the host once per call, as in the reference script.

The compute steps go through a small backend object so that the host logic (maps, splits,
ordering) can be exercised on CPU ranks with a checker backend supplied by the tests; the
default backend calls the C ABI and needs a CUDA device.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import _lib
from .ops import scale_k_padded


class CudaBackend:
    """The product path: every step is a call into the C ABI on torch's current stream."""

    def __init__(self):
        self.L = _lib.lib()

    @staticmethod
    def _stream(t: torch.Tensor) -> int:
        return torch.cuda.current_stream(t.device).cuda_stream

    def route(self, topk_ids, num_experts):
        t, k = topk_ids.shape
        dev = topk_ids.device
        pos = torch.empty((t, k), dtype=torch.int32, device=dev)
        seqlens = torch.empty(num_experts, dtype=torch.int32, device=dev)
        cu = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
        _lib.check(self.L.b200_nvfp4_moe_route(topk_ids.data_ptr(), pos.data_ptr(), seqlens.data_ptr(),
                                               cu.data_ptr(), t, k, num_experts, 0, self._stream(topk_ids)),
                   "moe_route")
        return pos, seqlens, cu

    def scatter_rows(self, src, pos, rows_out):
        out = torch.empty((rows_out, src.shape[1]), dtype=src.dtype, device=src.device)
        _lib.check(self.L.b200_nvfp4_moe_scatter_rows(out.data_ptr(), src.data_ptr(), pos.data_ptr(), pos.numel(),
                                                      pos.shape[1], src.shape[1] * src.element_size(),
                                                      self._stream(src)), "moe_scatter_rows")
        return out

    def gather_rows(self, src, index, rows_out):
        out = torch.empty((rows_out, src.shape[1]), dtype=src.dtype, device=src.device)
        if rows_out:
            _lib.check(self.L.b200_nvfp4_moe_gather_rows(out.data_ptr(), src.data_ptr(), index.data_ptr(), rows_out,
                                                         src.shape[1] * src.element_size(), self._stream(src)),
                       "moe_gather_rows")
        return out

    def quantize_gather(self, rows, row_map, seqlens, cu_seqlens, m_pad):
        r, hidden = row_map.numel(), rows.shape[1]
        e = seqlens.numel()
        packed = torch.empty((max(r, 1), hidden // 2), dtype=torch.uint8, device=rows.device)
        scales = torch.empty((e, m_pad * scale_k_padded(hidden)), dtype=torch.uint8, device=rows.device)
        if r:
            _lib.check(self.L.b200_nvfp4_moe_quantize_expert_gather(
                packed.data_ptr(), scales.data_ptr(), rows.data_ptr(), row_map.data_ptr(), seqlens.data_ptr(),
                cu_seqlens.data_ptr(), e, r, hidden, m_pad, int(rows.dtype == torch.bfloat16), 0,
                self._stream(rows)), "moe_quantize_expert_gather")
        return packed, scales

    def expert_moe(self, packed, scales, gate_up_w, gate_up_ws, down_w, down_ws, seqlens, cu_seqlens, rows, m_pad):
        hidden = packed.shape[1] * 2
        e, inter = gate_up_w.shape[0], gate_up_w.shape[1] // 2
        out = torch.empty((max(rows, 1), hidden), dtype=torch.float16, device=packed.device)
        if rows:
            need = self.L.b200_nvfp4_expert_moe_workspace_bytes(rows, hidden, inter, e, m_pad)
            ws = torch.empty(need, dtype=torch.uint8, device=packed.device)
            _lib.check(self.L.b200_nvfp4_expert_moe(
                out.data_ptr(), packed.data_ptr(), scales.data_ptr(), gate_up_w.data_ptr(), gate_up_ws.data_ptr(),
                down_w.data_ptr(), down_ws.data_ptr(), seqlens.data_ptr(), cu_seqlens.data_ptr(), ws.data_ptr(), need,
                rows, hidden, inter, e, m_pad, self._stream(packed)), "expert_moe")
        return out

    def reduce(self, rows, pos, weights, out_bf16):
        t, k = pos.shape
        hidden = rows.shape[1]
        out = torch.empty((t, hidden), dtype=torch.bfloat16 if out_bf16 else torch.float16, device=rows.device)
        _lib.check(self.L.b200_nvfp4_moe_reduce(out.data_ptr(), rows.data_ptr(), pos.data_ptr(), weights.data_ptr(),
                                                None, t, hidden, k, int(out_bf16), self._stream(rows)), "moe_reduce")
        return out


def expert_major_maps(counts: torch.Tensor, total: int):
    """counts[s, e] = rows rank s sent for local expert e (int64, on the compute device).

    The receive buffer is source-major (all of rank 0's rows, sorted by expert, then rank 1's
    ...). Returns (seqlens[e], cu_seqlens[e+1], row_map, inv_map): row_map[i] = receive-buffer
    row of expert-major row i (experts ascending, sources ascending inside an expert, send order
    inside a source) and inv_map its inverse.
    """
    w, e = counts.shape
    dev = counts.device
    seqlens = counts.sum(0)
    cu = torch.zeros(e + 1, dtype=torch.int64, device=dev)
    cu[1:] = torch.cumsum(seqlens, 0)
    src_base = torch.zeros(w, dtype=torch.int64, device=dev)
    src_base[1:] = torch.cumsum(counts.sum(1), 0)[:-1]
    recv_start = src_base[:, None] + torch.cumsum(counts, 1) - counts            # [w, e]
    em_start = cu[:-1][None, :] + torch.cumsum(counts, 0) - counts               # [w, e]
    # blocks in expert-major order: (e, s)
    lens = counts.t().reshape(-1)
    recv_s = recv_start.t().reshape(-1)
    em_s = em_start.t().reshape(-1)
    block = torch.repeat_interleave(torch.arange(w * e, device=dev), lens, output_size=total)
    idx = torch.arange(total, device=dev)
    row_map = (recv_s[block] + (idx - em_s[block])).to(torch.int32)
    inv_map = torch.empty(total, dtype=torch.int32, device=dev)
    inv_map[row_map.long()] = idx.to(torch.int32)
    return seqlens.to(torch.int32), cu.to(torch.int32), row_map, inv_map


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

    def _all_to_all_rows(self, send, send_splits, recv_splits):
        recv = torch.empty((sum(recv_splits), send.shape[1]), dtype=send.dtype, device=send.device)
        if self.world == 1:
            recv.copy_(send)
        else:
            dist.all_to_all_single(recv, send, recv_splits, send_splits, group=self.group)
        return recv

    @torch.no_grad()
    def forward(self, x, topk_ids, topk_weights, out_bf16: bool = True):
        w, e_local, be = self.world, self.e_local, self.backend
        t, k = topk_ids.shape
        total = t * k
        # 1. expert-major positions over ALL experts = (destination rank, expert, flat index) order
        pos, seqlens, _ = be.route(topk_ids, self.num_experts_total)
        send_counts = seqlens.view(w, e_local).to(torch.int64)
        # 2. per-expert counts to every destination rank
        recv_counts = torch.empty_like(send_counts)
        if w == 1:
            recv_counts.copy_(send_counts)
        else:
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        host = torch.cat((send_counts.sum(1), recv_counts.reshape(-1))).cpu()   # the one host read-back
        send_splits = host[:w].tolist()
        recv_host = host[w:].view(w, e_local)
        recv_splits = recv_host.sum(1).tolist()
        # 3. dispatch: token rows in send order, then the exchange
        send_rows = be.scatter_rows(x, pos, total)
        recv_rows = self._all_to_all_rows(send_rows, send_splits, recv_splits)
        self.last_bytes["dispatch"] = (total - send_splits[self.rank]) * x.shape[1] * x.element_size()
        # 4. local experts: permute + quantise, gate/up GEMM, SiLU*up + quantise, down GEMM
        rows = int(sum(recv_splits))
        seq_l, cu_l, row_map, inv_map = expert_major_maps(recv_counts, rows)
        max_rows = int(recv_host.sum(0).max()) if rows else 0
        m_pad = max(128, (max_rows + 127) // 128 * 128)
        packed, scales = be.quantize_gather(recv_rows, row_map, seq_l, cu_l, m_pad)
        y = be.expert_moe(packed, scales, self.gw, self.gws, self.dw, self.dws, seq_l, cu_l, rows, m_pad)
        # 5. combine: rows back in receive order, the exchange, weighted top-k sum at the source
        back = be.gather_rows(y, inv_map, rows)
        ret = self._all_to_all_rows(back, recv_splits, send_splits)
        self.last_bytes["combine"] = (rows - recv_splits[self.rank]) * y.shape[1] * y.element_size()
        return be.reduce(ret, pos, topk_weights, out_bf16)
