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

Two transports carry the records and the partial rows. "nccl": `all_to_all_single` (one host
read-back of the split sizes per call, as in the reference script). "p2p": no collective library
and no host read-back in the data path - every rank owns slotted receive / return buffers in
symmetric memory (torch.distributed._symmetric_memory maps them, CUDA IPC over NVLink) and the pack /
return kernels store straight into the peer's slots (b200_nvfp4_ep_dispatch_p2p / _ep_unpack_slots
/ _ep_reduce_return_p2p). The two hand-offs of a layer (records delivered, partial rows delivered)
are ordered by per-rank ready words (handoff="flags", the default): after its stores a rank
publishes the step's epoch into one word of every peer (b200_nvfp4_ep_publish_p2p, waits for
nobody), and the consuming kernels wait per source - the unpack kernel takes up the rows of source
s once s has published, so ranks that delivered early are unpacked while others are still sending,
and the final sum waits for the partial rows (b200_nvfp4_ep_unpack_slots_ready / _ep_sum_p2p).
With return_blocks > 1 the down projection runs as that many column blocks
(b200_nvfp4_grouped_gemm_columns) and the weighted sum + return stores of a finished block run on a
second stream beside the next block's GEMM (b200_nvfp4_ep_reduce_return_p2p_columns), so part of
the NVLink time of the return path hides behind tensor-core time.
handoff="barrier" separates the phases by two full cross-GPU barriers instead (this library's
b200_nvfp4_ep_barrier_p2p: epoch flags stored into the peers, a wait on the local ones). Every wait
is bounded: a rank that never arrives costs the others one time-out (about a second by default)
and shows in the device error word (_lib.device_error()), it cannot hang them. A layer whose call
raised or timed out on some rank is out of step with its peers (its step counter no longer matches
theirs): build a new one before the next call.

The compute steps go through a small backend object so that the host logic (splits, ordering,
the two exchanges) can be exercised on CPU ranks with a checker backend supplied by the tests;
the default backend calls the C ABI and needs a CUDA device.
"""
from __future__ import annotations

import ctypes
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


# Flag words of one rank: [0, 64) the barrier's, then world "records delivered" words (by source
# rank) and world "partial rows delivered" words (by expert rank).
BARRIER_WORDS = 64
FLAG_WORDS = 3 * BARRIER_WORDS


def ready_slot(which: str, world: int) -> int:
    return BARRIER_WORDS + (0 if which == "dispatch" else world)


def publish_ready(peer_flag, my_rank: int, world: int, which: str, step: int, device):
    stream = torch.cuda.current_stream(device).cuda_stream
    _lib.check(_lib.lib().b200_nvfp4_ep_publish_p2p(peer_flag, my_rank, world, ready_slot(which, world),
                                                    wrap_epoch(step), stream), "ep_publish_p2p")


def wrap_epoch(step: int) -> int:
    """The step counter as the int32 the kernels compare with wrap-around (seen - epoch >= 0)."""
    return (step + 2 ** 31) % 2 ** 32 - 2 ** 31


class _PeerBuffers:
    """Slotted receive / return buffers of one rank, visible to every peer (symmetric memory), and
    the flag words of this library's own cross-GPU barrier (b200_nvfp4_ep_barrier_p2p: peer stores
    of an epoch, a bounded wait on the local flags, a time-out reported through the device error
    word). torch's symmetric memory only maps the buffers; no library barrier runs per layer."""

    def __init__(self, group, world: int, slot_rows: int, hidden: int, topk: int, device, my_rank: int,
                 barrier_limit_cycles: int = 0):
        import torch.distributed._symmetric_memory as symm_mem
        self.world, self.slot_rows, self.hidden, self.topk = world, slot_rows, hidden, topk
        self.my_rank, self.limit = my_rank, int(barrier_limit_cycles)
        self.rb = record_bytes(hidden, topk)
        rows = world * slot_rows
        rec_bytes = rows * self.rb
        self.cnt_off = (rec_bytes + 255) // 256 * 256
        self.flag_off = self.cnt_off + 256
        self.ret_off = self.flag_off + 4 * FLAG_WORDS
        total = self.ret_off + rows * hidden * 2
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        group = group if group is not None else dist.group.WORLD
        self.handle = symm_mem.rendezvous(self.buf, group=group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        arr = ctypes.c_void_p * world
        self.peer_rec = arr(*ptrs)
        self.peer_cnt = arr(*[p + self.cnt_off for p in ptrs])
        self.peer_flag = arr(*[p + self.flag_off for p in ptrs])
        self.peer_ret = arr(*[p + self.ret_off for p in ptrs])
        self.rec = self.buf[:rec_bytes].view(rows, self.rb)
        self.cnt = self.buf[self.cnt_off:self.cnt_off + 4 * world].view(torch.int32)
        self.ret = self.buf[self.ret_off:total].view(torch.float16).view(rows, hidden)
        self.flags = self.buf[self.flag_off:self.flag_off + 4 * FLAG_WORDS].view(torch.int32)
        self.epoch = 0          # barrier epochs
        self.step = 0           # ready-word epochs: one per layer call
        self.buf.zero_()
        # set-up only: no rank may publish an epoch before every rank has cleared its flags
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def barrier(self):
        self.epoch += 1
        stream = torch.cuda.current_stream(self.buf.device).cuda_stream
        _lib.check(_lib.lib().b200_nvfp4_ep_barrier_p2p(self.peer_flag, self.my_rank, self.world, self.epoch,
                                                        self.limit, stream), "ep_barrier_p2p")

    def publish(self, which: str):
        """Tell every peer that this rank's stores of the current step's `which` phase ("dispatch" or
        "return"), issued before this call on the current stream, are complete."""
        publish_ready(self.peer_flag, self.my_rank, self.world, which, self.step, self.buf.device)

    def ready_ptr(self, which: str) -> int:
        return self.flags.data_ptr() + 4 * ready_slot(which, self.world)


class ExpertParallelMoE:
    """One MoE layer whose experts are sharded over the ranks of `group`.

    gate_up_weight [E_local, 2I, H/2], down_weight [E_local, H, I/2] (packed E2M1) and their
    scale regions are this rank's experts. forward() takes this rank's tokens (BF16 or FP16
    [T, H]), their top-k expert ids over all E experts and the route weights, and returns
    [T, H] (BF16 by default).
    """

    def __init__(self, gate_up_weight, gate_up_weight_scale, down_weight, down_weight_scale, num_experts_total: int,
                 group: Optional[dist.ProcessGroup] = None, backend=None, transport: str = "nccl",
                 max_tokens: int = 0, num_topk: int = 0, emulate=None, barrier_limit_cycles: int = 0,
                 handoff: str = "flags", return_blocks: int = 0):
        self.gw, self.gws, self.dw, self.dws = gate_up_weight, gate_up_weight_scale, down_weight, down_weight_scale
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if emulate is not None:
            # (world, rank, peers): one process plays several ranks of the p2p transport, with a
            # peers object whose pointer tables address the other emulated ranks' buffers
            self.world, self.rank = int(emulate[0]), int(emulate[1])
        self.num_experts_total = int(num_experts_total)
        self.e_local = gate_up_weight.shape[0]
        if self.e_local * self.world != self.num_experts_total:
            raise ValueError("num_experts_total must equal world_size * local experts")
        self.backend = backend if backend is not None else CudaBackend()
        self.last_bytes = {"dispatch": 0, "combine": 0}
        self._ones = None
        if transport not in ("nccl", "p2p"):
            raise ValueError("transport must be 'nccl' or 'p2p'")
        if handoff not in ("flags", "barrier"):
            raise ValueError("handoff must be 'flags' or 'barrier'")
        self.transport, self.handoff = transport, handoff
        self.wait_limit = int(barrier_limit_cycles)
        # p2p transport: the down projection in this many column blocks; the partial rows of a
        # finished block go back to their sources on a second stream while the next one is computed
        # (0 = choose: two blocks where the slots of a rank hold 16384 rows or more - measured with
        # T = 4096 per rank, P50 per layer: 4 GPUs 1.45 -> 1.35 ms, 8 GPUs 1.69 -> 1.53 ms; with 4096
        # tokens in total one block is faster (4 GPUs 0.577 against 0.588 ms, 8 GPUs 0.406 against
        # 0.412), and on 2 GPUs the return stores are too short to matter)
        self.return_blocks = int(return_blocks)
        hidden_size = gate_up_weight.shape[2] * 2
        if self.return_blocks == 0:
            big = transport == "p2p" and emulate is None and self.world * int(max_tokens) >= 16384
            self.return_blocks = 2 if big and hidden_size % 256 == 0 else 1
        if self.return_blocks < 1 or hidden_size % (128 * self.return_blocks) != 0:
            raise ValueError("return_blocks must divide the hidden size into multiples of 128 columns")
        self._side = None
        self.peers = None
        if emulate is not None:
            self.peers = emulate[2]
        elif transport == "p2p":
            if max_tokens <= 0 or num_topk <= 0:
                raise ValueError("the p2p transport needs max_tokens (tokens per rank per call) and num_topk")
            hidden = gate_up_weight.shape[2] * 2
            self.peers = _PeerBuffers(group, self.world, int(max_tokens), hidden, int(num_topk), gate_up_weight.device,
                                      self.rank, barrier_limit_cycles)

    def _all_to_all_rows(self, send, send_splits, recv_splits):
        recv = torch.empty((sum(recv_splits), send.shape[1]), dtype=send.dtype, device=send.device)
        if self.world == 1:
            recv.copy_(send)
        else:
            dist.all_to_all_single(recv, send, recv_splits, send_splits, group=self.group)
        return recv

    def _p2p_workspace(self, rows: int, hidden: int, k: int, device):
        """Intermediates of the routed layer over all slot rows, allocated once per layer: the slots
        have a fixed capacity, so the sizes never change."""
        if getattr(self, "_ws", None) is not None:
            return self._ws
        inter = self.gw.shape[1] // 2
        total = rows * k
        in_pad = (rows + 127) // 128 * 128
        m_pad = in_pad          # a token reaches an expert at most once: no expert sees more rows than there are slots
        u8 = dict(dtype=torch.uint8, device=device)
        i32 = dict(dtype=torch.int32, device=device)
        f16 = dict(dtype=torch.float16, device=device)
        self._ws = {
            "inter": inter, "m_pad": m_pad, "in_pad": in_pad,
            "xq": torch.empty((rows, hidden // 2), **u8), "xs": torch.empty(in_pad * scale_k_padded(hidden), **u8),
            "ids": torch.empty((rows, k), **i32), "wts": torch.empty((rows, k), dtype=torch.float32, device=device),
            "gin": torch.empty((total, hidden // 2), **u8),
            "gin_s": torch.empty((self.e_local, m_pad * scale_k_padded(hidden)), **u8),
            "gout": None,    # FP16 gate/up product: only the unfused fallback needs it (allocated there)
            "din": torch.empty((total, inter // 2), **u8),
            "din_s": torch.empty((self.e_local, m_pad * scale_k_padded(inter)), **u8),
            "dout": torch.empty((total, hidden), **f16), "pos": torch.empty((rows, k), **i32),
            "seq": torch.empty(self.e_local, **i32), "cu": torch.empty(self.e_local + 1, **i32),
        }
        return self._ws

    # The p2p layer in three phases. With handoff="flags" a phase ends by publishing its ready word
    # and the next one waits for the words it needs inside its first kernel; with "barrier" every
    # rank passes a barrier between them. They are separate methods so that a single process can step
    # several emulated ranks through them in turn.
    @torch.no_grad()
    def p2p_dispatch(self, x, topk_ids, topk_weights):
        """Phase 1: quantise this rank's tokens and store their records into the destination ranks'
        slots. Returns ret_pos [T, world]: where each token's partial rows will come back."""
        w, be, pb = self.world, self.backend, self.peers
        t, hidden = x.shape
        k = topk_ids.shape[1]
        if t > pb.slot_rows or k != pb.topk or hidden != pb.hidden:
            raise ValueError("call does not fit the peer buffers this layer was built with")
        L = _lib.lib()
        stream = torch.cuda.current_stream(x.device).cuda_stream
        dest = be.dest_ranks(topk_ids, self.e_local, w)
        send_pos, send_counts, send_cu = be.route(dest, w)
        ret_pos = torch.empty((t, w), dtype=torch.int32, device=x.device)
        _lib.check(L.b200_nvfp4_ep_dispatch_p2p(pb.peer_rec, pb.peer_cnt, ret_pos.data_ptr(), x.data_ptr(),
                                                topk_ids.data_ptr(), topk_weights.data_ptr(), send_pos.data_ptr(),
                                                send_counts.data_ptr(), send_cu.data_ptr(), self.rank, w, pb.slot_rows,
                                                t, hidden, k, int(x.dtype == torch.bfloat16), stream), "ep_dispatch_p2p")
        if self.handoff == "flags":
            pb.step += 1
            pb.publish("dispatch")
        return ret_pos

    @torch.no_grad()
    def p2p_compute_and_return(self, mark=None):
        """Phase 2: the routed layer over this rank's experts on everything its slots received, the
        partial rows stored into the source ranks' return slots."""
        w, pb = self.world, self.peers
        hidden, k = pb.hidden, pb.topk
        L = _lib.lib()
        device = pb.rec.device
        stream = torch.cuda.current_stream(device).cuda_stream
        rows = w * pb.slot_rows
        ws = self._p2p_workspace(rows, hidden, k, device)
        flags = self.handoff == "flags"
        _lib.check(L.b200_nvfp4_ep_unpack_slots_ready(
            ws["xq"].data_ptr(), ws["xs"].data_ptr(), ws["ids"].data_ptr(), ws["wts"].data_ptr(), pb.rec.data_ptr(),
            pb.cnt.data_ptr(), w, pb.slot_rows, hidden, k, pb.ready_ptr("dispatch") if flags else None,
            wrap_epoch(pb.step) if flags else 0, self.wait_limit, stream), "ep_unpack_slots_ready")
        if mark is not None and flags:
            mark("wait_records_and_unpack")
        # the routed layer stage by stage (what b200_nvfp4_fused_moe runs), with its last step - the
        # weighted sum over a token's local experts - storing straight into the source ranks' slots
        inter, total, m_pad = ws["inter"], rows * k, ws["m_pad"]
        avg = max(1, total // self.num_experts_total)
        _lib.check(L.b200_nvfp4_moe_count_and_gather(
            ws["gin"].data_ptr(), ws["gin_s"].data_ptr(), ws["xq"].data_ptr(), ws["xs"].data_ptr(), ws["ids"].data_ptr(),
            ws["pos"].data_ptr(), ws["seq"].data_ptr(), ws["cu"].data_ptr(), rows, hidden, k, self.e_local, self.rank,
            ws["in_pad"], m_pad, 0, stream), "moe_count_and_gather")
        # gate/up projection with SiLU * up and the quantisation in its epilogue; the two separate steps
        # only where the fused kernel does not cover the intermediate size (same bytes either way)
        status = L.b200_nvfp4_grouped_gemm_swiglu_quant(
            ws["din"].data_ptr(), ws["din_s"].data_ptr(), ws["gin"].data_ptr(), self.gw.data_ptr(), ws["seq"].data_ptr(),
            ws["cu"].data_ptr(), ws["gin_s"].data_ptr(), self.gws.data_ptr(), None, None, self.e_local, total, inter,
            hidden, m_pad, m_pad, avg, stream)
        if status == _lib.STATUS_NOT_SUPPORTED:
            if ws["gout"] is None:
                ws["gout"] = torch.empty((total, 2 * inter), dtype=torch.float16, device=device)
            _lib.check(L.b200_nvfp4_grouped_gemm(
                ws["gout"].data_ptr(), ws["gin"].data_ptr(), self.gw.data_ptr(), ws["seq"].data_ptr(), ws["cu"].data_ptr(),
                ws["gin_s"].data_ptr(), self.gws.data_ptr(), None, None, None, self.e_local, total, 2 * inter, hidden,
                m_pad, avg, 1, None, stream), "grouped_gemm (gate/up)")
            _lib.check(L.b200_nvfp4_moe_act_mul_and_quant(
                ws["din"].data_ptr(), ws["din_s"].data_ptr(), ws["gout"].data_ptr(), ws["seq"].data_ptr(),
                ws["cu"].data_ptr(), self.e_local, total, m_pad, inter, 0, stream), "moe_act_mul_and_quant")
        else:
            _lib.check(status, "grouped_gemm_swiglu_quant")
        nb = self.return_blocks
        if nb == 1:
            _lib.check(L.b200_nvfp4_grouped_gemm(
                ws["dout"].data_ptr(), ws["din"].data_ptr(), self.dw.data_ptr(), ws["seq"].data_ptr(),
                ws["cu"].data_ptr(), ws["din_s"].data_ptr(), self.dws.data_ptr(), None, None, None, self.e_local, total,
                hidden, inter, m_pad, avg, 1, None, stream), "grouped_gemm (down)")
            if mark is not None:
                mark("routed_layer")
            _lib.check(L.b200_nvfp4_ep_reduce_return_p2p(pb.peer_ret, ws["dout"].data_ptr(), ws["pos"].data_ptr(),
                                                         ws["wts"].data_ptr(), pb.cnt.data_ptr(), self.rank, w,
                                                         pb.slot_rows, hidden, k, stream), "ep_reduce_return_p2p")
        else:
            # column blocks of the down projection on this stream; the weighted sum + return stores of
            # block b on a second stream as soon as block b is complete, beside the GEMM of block b + 1
            main = torch.cuda.current_stream(device)
            if self._side is None:
                self._side = (torch.cuda.Stream(device), [torch.cuda.Event() for _ in range(nb)])
            side, events = self._side
            width = hidden // nb

            def reduce_return(block, on):
                _lib.check(L.b200_nvfp4_ep_reduce_return_p2p_columns(
                    pb.peer_ret, ws["dout"].data_ptr(), ws["pos"].data_ptr(), ws["wts"].data_ptr(), pb.cnt.data_ptr(),
                    self.rank, w, pb.slot_rows, hidden, k, block * width, width, on.cuda_stream),
                    "ep_reduce_return_p2p_columns")

            for b in range(nb):
                _lib.check(L.b200_nvfp4_grouped_gemm_columns(
                    ws["dout"].data_ptr(), ws["din"].data_ptr(), self.dw.data_ptr(), ws["seq"].data_ptr(),
                    ws["cu"].data_ptr(), ws["din_s"].data_ptr(), self.dws.data_ptr(), self.e_local, total, hidden, inter,
                    m_pad, avg, None, b * width, width, stream), "grouped_gemm_columns (down)")
                if b < nb - 1:
                    events[b].record(main)
                    side.wait_event(events[b])
                    reduce_return(b, side)
            if mark is not None:
                mark("routed_layer")
            reduce_return(nb - 1, main)
            events[nb - 1].record(side)
            main.wait_event(events[nb - 1])
        if flags:
            pb.publish("return")
        if mark is not None:
            mark("reduce_and_return")

    @torch.no_grad()
    def p2p_finish(self, ret_pos, out_bf16: bool = True):
        """Phase 3: sum the partial rows that came back, in ascending rank order."""
        t, w = ret_pos.shape
        pb = self.peers
        if self.handoff == "flags":
            out = torch.empty((t, pb.hidden), dtype=torch.bfloat16 if out_bf16 else torch.float16, device=ret_pos.device)
            stream = torch.cuda.current_stream(ret_pos.device).cuda_stream
            _lib.check(_lib.lib().b200_nvfp4_ep_sum_p2p(out.data_ptr(), pb.ret.data_ptr(), ret_pos.data_ptr(), t,
                                                        pb.hidden, w, int(out_bf16), pb.ready_ptr("return"),
                                                        wrap_epoch(pb.step), self.wait_limit, stream), "ep_sum_p2p")
            return out
        if self._ones is None or self._ones.shape != (t, w) or self._ones.device != ret_pos.device:
            self._ones = torch.ones((t, w), dtype=torch.float32, device=ret_pos.device)
        return self.backend.reduce(self.peers.ret, ret_pos, self._ones, out_bf16)

    def _forward_p2p(self, x, topk_ids, topk_weights, out_bf16: bool, phase_events=None):
        def mark(name):
            if phase_events is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                phase_events.append((name, ev))

        mark("start")
        ret_pos = self.p2p_dispatch(x, topk_ids, topk_weights)
        mark("dispatch")
        if self.handoff == "barrier":
            self.peers.barrier()
            mark("barrier_after_dispatch")
        self.p2p_compute_and_return(mark)
        if self.handoff == "barrier":
            self.peers.barrier()
            mark("barrier_after_return")
        out = self.p2p_finish(ret_pos, out_bf16)
        mark("sum")
        return out

    @torch.no_grad()
    def forward(self, x, topk_ids, topk_weights, out_bf16: bool = True, phase_events=None):
        """phase_events: optional list; the p2p transport appends (phase name, CUDA event) pairs
        recorded on the current stream after each phase of the layer."""
        if self.transport == "p2p":
            return self._forward_p2p(x, topk_ids, topk_weights, out_bf16, phase_events)
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
