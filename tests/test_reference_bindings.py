"""The reference's own torch bindings (bindings/gemm_ops.cu, grouped_gemm_ops.cpp,
fused_moe_ops.cpp) compiled UNCHANGED against this repository's include/sm120_nvfp4/*.hpp and
linked to its library (recipe: oracle/build.py:build_ref_bindings, output oracle/_ref/, made in
the build container where the reference checkout exists; the built file travels, the sources do
not). The CPU test loads the result in a fresh interpreter and checks the registered schemas; the
GPU test calls the reference's ops - its argument checks, its output allocation, its workspace
carve - on this library's kernels and compares with the known answers the reference's own tests
hold (tests/python/test_gemm.py:39-68 all-ones -> K; test_fused_moe.py:96-101 -> 33792;
test_grouped_gemm.py:23-46 group sizes [0, 1, 127, 129]).

The child process never imports sm120_nvfp4_b200.ops: that module registers the same operator
names from Python, and one process can hold only one definition."""
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _library():
    sys.path.insert(0, str(ROOT))
    from oracle import build as oracle_build
    from sm120_nvfp4_b200 import build as lib_build
    lib_build.build()
    try:
        return oracle_build.build_ref_bindings()
    except Exception as exc:      # reference present but it does not compile against our headers: a failure
        pytest.fail(f"the reference bindings do not build against include/sm120_nvfp4: {exc}")


def _child(code: str, timeout=600):
    res = subprocess.run([sys.executable, "-c", textwrap.dedent(code)], capture_output=True, text=True, timeout=timeout,
                         cwd=str(ROOT))
    assert res.returncode == 0 and "PASS" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]


SCHEMAS = {
    "gemm": "sm120_nvfp4::gemm(Tensor a, Tensor b, Tensor sfa, Tensor sfb) -> Tensor",
    "cute_gemm": "sm120_nvfp4::cute_gemm(Tensor a, Tensor b, Tensor sfa, Tensor sfb) -> Tensor",
    "cutlass_gemm": "sm120_nvfp4::cutlass_gemm(Tensor a, Tensor b, Tensor sfa, Tensor sfb) -> Tensor",
    "grouped_gemm": "sm120_nvfp4::grouped_gemm(Tensor x, Tensor weight, Tensor seqlens, Tensor cu_seqlens, "
                    "Tensor x_scale, Tensor w_scale, int num_seq_per_group_avg, Tensor? output, Tensor? tma_desc) -> Tensor",
    "fused_moe": "sm120_nvfp4::fused_moe(Tensor input, Tensor input_scale, Tensor gate_up_weight, "
                 "Tensor gate_up_weight_scale, Tensor down_weight, Tensor down_weight_scale, Tensor topk_ids, "
                 "Tensor topk_scale, Tensor? shared_output, int rank_ep, int num_expert_total, Tensor? output) -> Tensor",
    "quantize_expert": "sm120_nvfp4::quantize_expert(Tensor input, Tensor seqlens, Tensor cu_seqlens, int scale_m_pad, "
                       "Tensor? output, Tensor? output_scale) -> (Tensor, Tensor)",
    "expert_moe": "sm120_nvfp4::expert_moe(Tensor input, Tensor input_scale, Tensor gate_up_weight, "
                  "Tensor gate_up_weight_scale, Tensor down_weight, Tensor down_weight_scale, Tensor seqlens, "
                  "Tensor cu_seqlens, Tensor? output, Tensor? workspace) -> Tensor",
}


def test_reference_bindings_build_and_register_their_schemas():
    lib = _library()
    if lib is None:
        pytest.skip("no reference checkout and no earlier build of oracle/_ref/libref_bindings.so")
    _child(f"""
        import torch
        torch.ops.load_library({str(lib)!r})
        want = {SCHEMAS!r}
        for name, schema in want.items():
            got = str(getattr(torch.ops.sm120_nvfp4, name).default._schema)
            assert got == schema, (name, got)
        print("PASS")
    """)


@pytest.mark.gpu
def test_reference_bindings_run_on_this_library():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    lib = _library()
    if lib is None:
        pytest.skip("oracle/_ref/libref_bindings.so was not built (no reference checkout at build time)")
    _child(f"""
        import torch
        torch.ops.load_library({str(lib)!r})
        ops = torch.ops.sm120_nvfp4
        dev = "cuda"
        u8 = dict(dtype=torch.uint8, device=dev)

        def skp(k):
            return ((k + 15) // 16 + 3) // 4 * 4

        # all-ones GEMM through every reference entry: payload 0x22 = (1.0, 1.0), scale 0x38 = 1.0
        for m, n, k in ((16, 256, 512), (128, 512, 1024), (256, 256, 512)):
            a = torch.full((m, k // 2), 0x22, **u8)
            b = torch.full((n, k // 2), 0x22, **u8)
            sfa = torch.full(((m + 127) // 128 * 128 * skp(k),), 0x38, **u8)
            sfb = torch.full(((n + 127) // 128 * 128 * skp(k),), 0x38, **u8)
            for op in (ops.gemm, ops.cute_gemm, ops.cutlass_gemm):
                out = op(a, b, sfa, sfb)
                assert out.dtype == torch.float16 and tuple(out.shape) == (m, n)
                assert bool((out == k).all()), (m, n, k)
        # the reference's argument checks are the ones that run
        try:
            ops.gemm(a.float(), b, sfa, sfb)
            raise SystemExit("dtype check did not fire")
        except RuntimeError as exc:
            assert "packed storage" in str(exc)

        # grouped GEMM, group sizes [0, 1, 127, 129] (unit data: every valid output is K)
        counts = [0, 1, 127, 129]
        g, n, k, m_pad = len(counts), 256, 256, 256
        total = sum(counts)
        x = torch.full((total, k // 2), 0x22, **u8)
        w = torch.full((g, n, k // 2), 0x22, **u8)
        xs = torch.full((g, m_pad * skp(k)), 0x38, **u8)
        ws = torch.full((g, n * skp(k)), 0x38, **u8)
        seq = torch.tensor(counts, dtype=torch.int32, device=dev)
        cu = torch.tensor([0, 0, 1, 128, 257], dtype=torch.int32, device=dev)
        y = ops.grouped_gemm(x, w, seq, cu, xs, ws, 64, None, None)
        assert tuple(y.shape) == (total, n) and bool((y == k).all())

        # fused MoE known answer: 0x11 payloads (0.5), unit scales -> 33792 everywhere (+ shared 2.0)
        tokens, experts, hidden, inter = 4, 2, 128, 64
        xq = torch.full((tokens, hidden // 2), 0x11, **u8)
        gw = torch.full((experts, 2 * inter, hidden // 2), 0x11, **u8)
        dw = torch.full((experts, hidden, inter // 2), 0x11, **u8)
        xsc = torch.full((128 * skp(hidden),), 0x38, **u8)
        gs = torch.full((experts, 128 * skp(hidden)), 0x38, **u8)
        ds = torch.full((experts, 128 * skp(inter)), 0x38, **u8)
        ids = torch.tensor([[0, 1], [1, 0], [0, 1], [1, 0]], dtype=torch.int32, device=dev)
        wt = torch.tensor([[0.25, 0.75], [0.6, 0.4], [0.5, 0.5], [0.2, 0.8]], dtype=torch.float32, device=dev)
        out = ops.fused_moe(xq, xsc, gw, gs, dw, ds, ids, wt, None, 0, experts, None)
        torch.cuda.synchronize()
        assert tuple(out.shape) == (tokens, hidden) and bool((out == 33792).all()), out[0, :4]

        # expert_moe (the DeepEP-compatible entry) on the same data, rows already expert-major
        seq2 = torch.tensor([4, 4], dtype=torch.int32, device=dev)
        cu2 = torch.tensor([0, 4, 8], dtype=torch.int32, device=dev)
        xrows = torch.full((8, hidden // 2), 0x11, **u8)
        xrows_s = torch.full((experts, 128 * skp(hidden)), 0x38, **u8)
        rows = ops.expert_moe(xrows, xrows_s, gw, gs, dw, ds, seq2, cu2, None, None)
        torch.cuda.synchronize()
        assert tuple(rows.shape) == (8, hidden) and bool((rows == 33792).all()), rows[0, :4]

        # quantize_expert against the CPU oracle (payload bytes and the scale bytes of live rows)
        import sys
        import numpy as np
        sys.path.insert(0, {str(ROOT)!r})
        import oracle
        g = torch.Generator().manual_seed(5)
        xb = torch.randn((8, hidden), generator=g).to(torch.bfloat16)
        packed, scales = ops.quantize_expert(xb.to(dev), seq2, cu2, 128, None, None)
        xbits = xb.view(torch.int16).numpy().view(np.uint16)
        want_p, want_s = oracle.quantize_expert(xbits, [4, 4], [0, 4, 8], 128, True)
        assert np.array_equal(packed.cpu().numpy(), want_p)
        got_s = scales.cpu().numpy().reshape(experts, -1)
        want_s = np.asarray(want_s).reshape(experts, -1)
        nkb = hidden // 16
        r = np.repeat(np.arange(4, dtype=np.int32), nkb)
        kb = np.tile(np.arange(nkb, dtype=np.int32), 4)
        off = oracle.sf_offsets(r, kb, hidden)
        assert np.array_equal(got_s[:, off], want_s[:, off])
        print("PASS")
    """)
