"""Generate the committed golden fixtures in this folder from the reference.

Run once where the reference checkout is mounted (it is not needed at test
time):

    python tests/golden/make_golden.py

What comes from the reference itself:
  * quantizer.npz   - the torch quantiser restatement the reference uses as its
                      own analytic check (benchmarks/benchmark_moe_ops.py:18-29,
                      function `quantized_reference`) is loaded from the
                      reference file by name and executed on seeded BF16 input
                      that covers zero blocks, tiny blocks, huge blocks and
                      exact rounding ties.
  * sf_layout.npz   - byte offsets returned by the reference's own
                      src/fused_moe/scale_layout.cuh (sfa_offset / sfb_offset),
                      compiled by oracle/build.py, at seeded coordinates.
  * codecs.npz      - cutlass::float_ue4m3_t / float_e2m1_t and the CUDA
                      toolkit's e2m1 / e4m3 host conversions at seeded floats
                      plus every rounding boundary.
  * dyadic_gemm.npz - the exact-equality construction of
                      tests/python/test_gemm.py:17-37 (random payload bytes,
                      scales 0x18 / 0x20, expected = dequant-matmul in FP32
                      rounded to FP16) evaluated with torch on the CPU, and the
                      grouped variant of tests/python/test_grouped_gemm.py:17-52.
"""
from __future__ import annotations

import ast
import os
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
# the reference checkout: NVFP4_REFERENCE_DIR, else a directory named "reference" beside this repository
REFERENCE = Path(os.environ.get("NVFP4_REFERENCE_DIR", ROOT.parent / "reference"))
OUT = Path(__file__).resolve().parent


def load_reference_function(path: Path, name: str):
    tree = ast.parse(path.read_text())
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            module = ast.Module(body=[node], type_ignores=[])
            namespace = {"torch": torch}
            exec(compile(module, str(path), "exec"), namespace)
            return namespace[name]
    raise KeyError(name)


def make_quantizer():
    fn = load_reference_function(REFERENCE / "benchmarks" / "benchmark_moe_ops.py",
                                 "quantized_reference")
    g = torch.Generator().manual_seed(20260)
    rows, hidden = 24, 256
    x = torch.randn(rows, hidden, generator=g) * 0.25
    x[1] *= 1e-4                     # tiny blocks: subnormal UE4M3 scales
    x[2] *= 4000.0                   # large blocks
    x[3, :32] = 0.0                  # zero blocks
    x[4] *= 1e-7                     # scale underflows to the raw-1 rule
    x[5, :16] = torch.tensor([6., 5., 4., 3.5, 3., 2.5, 2., 1.75, 1.5, 1.25, 1., .75, .5, .25, 0., -5.])
    x[6] *= 60000.0                  # scale saturation region (amax/6 > 448 for some blocks)
    xb = x.bfloat16()
    expected = fn(xb)                # dequantised FP32, same shape
    np.savez_compressed(OUT / "quantizer.npz",
                        input_bf16_bits=xb.view(torch.int16).numpy().view(np.uint16),
                        expected_dequant=expected.numpy().astype(np.float32))


def make_layout_and_codecs():
    import oracle
    R = oracle.ref()
    assert R is not None, "reference shim not buildable here"
    rng = np.random.default_rng(7)
    rows_l, kb_l, mpad_l, k_l, sfa_l, sfb_l = [], [], [], [], [], []
    for m_pad in (128, 256, 384, 1024):
        for k in (32, 80, 128, 512, 2048, 7168, 8192):
            nkb = (k + 15) // 16
            for _ in range(64):
                r = int(rng.integers(0, m_pad))
                kb = int(rng.integers(0, nkb))
                rows_l.append(r); kb_l.append(kb); mpad_l.append(m_pad); k_l.append(k)
                sfa_l.append(R.ref_sfa_offset(r, kb, m_pad, k))
                sfb_l.append(R.ref_sfb_offset(r, kb, m_pad, k))
    np.savez_compressed(OUT / "sf_layout.npz", row=np.array(rows_l, np.int32),
                        k_block=np.array(kb_l, np.int32), m_pad=np.array(mpad_l, np.int32),
                        k=np.array(k_l, np.int32), sfa=np.array(sfa_l, np.int64),
                        sfb=np.array(sfb_l, np.int64))

    vals = list(rng.normal(size=2000).astype(np.float32) * 3)
    vals += list((rng.random(2000).astype(np.float32) * 500))
    vals += list(np.exp(rng.uniform(-25, 7, 4000)).astype(np.float32))
    # every midpoint between adjacent UE4M3 codes and adjacent E2M1 codes, +-1 ulp
    dec = [R.ref_cutlass_ue4m3_decode(b) for b in range(0x7f)]
    for lo, hi in zip(dec[:-1], dec[1:]):
        mid = np.float32((np.float64(lo) + np.float64(hi)) / 2)
        vals += [mid, np.nextafter(mid, np.float32(0)), np.nextafter(mid, np.float32(1e9))]
    for mid in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, 0.0):
        m32 = np.float32(mid)
        vals += [m32, np.nextafter(m32, np.float32(0)), np.nextafter(m32, np.float32(1e9)), -m32]
    vals += [448.0, 464.0, 480.0, 1e9, 2.0 ** -9, 2.0 ** -10, 2.0 ** -11, 3 * 2.0 ** -11]
    v = np.array(vals, np.float32)
    np.savez_compressed(
        OUT / "codecs.npz", value=v,
        cutlass_ue4m3=np.array([R.ref_cutlass_ue4m3_encode(float(abs(x))) for x in v], np.uint8),
        cuda_e4m3=np.array([R.ref_cuda_e4m3_encode(float(abs(x))) for x in v], np.uint8),
        cutlass_e2m1=np.array([R.ref_cutlass_e2m1_encode(float(x)) for x in v], np.uint8),
        cuda_e2m1=np.array([R.ref_cuda_e2m1_encode(float(x)) for x in v], np.uint8),
        ue4m3_table=np.array(dec, np.float32),
        e2m1_table=np.array([R.ref_cutlass_e2m1_decode(b) for b in range(16)], np.float32))


def make_dyadic():
    levels = torch.tensor([0., .5, 1., 1.5, 2., 3., 4., 6., -0., -.5, -1., -1.5, -2., -3., -4., -6.])

    def decode(packed):
        return levels[torch.stack((packed & 15, packed >> 4), -1).flatten(-2).long()]

    out = {}
    g = torch.Generator().manual_seed(920)
    n, k = 256, 512
    for m in (7, 128, 256):
        a = torch.randint(256, (m, k // 2), dtype=torch.uint8, generator=g)
        b = torch.randint(256, (n, k // 2), dtype=torch.uint8, generator=g)
        expected = ((decode(a) * .0625) @ (decode(b) * .125).T).half()
        out[f"a_{m}"] = a.numpy(); out[f"b_{m}"] = b.numpy()
        out[f"expected_{m}"] = expected.numpy()
    g = torch.Generator().manual_seed(921)
    groups, rows, n, k, pad = 4, 257, 128, 128, 256
    x = torch.randint(256, (rows, k // 2), dtype=torch.uint8, generator=g)
    weight = torch.randint(256, (groups, n, k // 2), dtype=torch.uint8, generator=g)
    codes = torch.tensor([0x10, 0x18, 0x20, 0x28], dtype=torch.uint8)
    out["gx"] = x.numpy(); out["gw"] = weight.numpy(); out["gcodes"] = codes.numpy()
    for idx, counts in enumerate(([0, 1, 127, 129], [129, 0, 1, 127])):
        prefix = [0]
        for c in counts:
            prefix.append(prefix[-1] + c)
        expected = torch.zeros((rows, n), dtype=torch.float16)
        for group in range(groups):
            begin, end = prefix[group:group + 2]
            aa = decode(x[begin:end]) * codes[group:group + 1].view(torch.float8_e4m3fn).float()
            bb = decode(weight[group]) * codes[3 - group:4 - group].view(torch.float8_e4m3fn).float()
            expected[begin:end] = (aa @ bb.T).half()
        out[f"gcounts_{idx}"] = np.array(counts, np.int32)
        out[f"gexpected_{idx}"] = expected.numpy()
    np.savez_compressed(OUT / "dyadic_gemm.npz", **out)


if __name__ == "__main__":
    make_quantizer()
    make_layout_and_codecs()
    make_dyadic()
    print("wrote", sorted(p.name for p in OUT.glob("*.npz")))
