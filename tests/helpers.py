"""Shared helpers of the tests: seeded synthetic NVFP4 data and the parity gates."""
from __future__ import annotations

import numpy as np

import oracle


def randn_quantized(rows: int, k: int, seed: int, std: float = 1.0):
    """Seeded N(0, std^2) FP32 [rows, k] quantised to NVFP4 by the oracle's quantiser."""
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((rows, k), dtype=np.float32) * np.float32(std))
    return oracle.quantize_rows(x)


def fp16_ulp(y: np.ndarray) -> np.ndarray:
    """Spacing of FP16 at |y| (FP32 array in, FP32 out); subnormal spacing below 2^-14."""
    a = np.abs(y.astype(np.float32))
    e = np.floor(np.log2(np.maximum(a, 2.0 ** -14)))
    return (2.0 ** (e - 10)).astype(np.float32)


def check_gemm_parity(got: np.ndarray, ref32: np.ndarray, rowmax: np.ndarray | None = None):
    """The GEMM gate: relative Frobenius error <= 1e-3 and, per element,
    |diff| <= 2 FP16 ulp(ref) + 1e-3 * max|ref| of the row. For FP16 outputs also: at least 99 % of
    the elements are exactly the oracle's FP32 value rounded to FP16 (measured on B200: 100 % at every
    full-size configuration, K = 8192 included - the accumulation order inside the tensor core does
    not show at FP16 precision)."""
    if got.dtype == np.float16 and got.size:
        exact = float((got == ref32.astype(np.float32).astype(np.float16)).mean())
        assert exact >= 0.99, f"only {exact:.4f} of the FP16 outputs equal the rounded oracle value"
    got = got.astype(np.float32)
    ref32 = ref32.astype(np.float32)
    assert np.isfinite(got).all(), "non-finite output"
    num = np.linalg.norm((got - ref32).astype(np.float64))
    den = max(np.linalg.norm(ref32.astype(np.float64)), 1e-30)
    frob = num / den
    if rowmax is None:
        rowmax = np.abs(ref32).max(axis=1)
    tol = 2.0 * fp16_ulp(ref32) + 1e-3 * rowmax[:, None]
    worst = float((np.abs(got - ref32) / tol).max()) if got.size else 0.0
    assert frob <= 1e-3, f"relative Frobenius error {frob:.3e} > 1e-3"
    assert worst <= 1.0, f"per-element gate exceeded by factor {worst:.3f}"
    return frob, worst


def topk_routing(num_tokens: int, num_experts: int, topk: int, seed: int):
    """Router of the DeepSeek-shaped config: logits N(0,1), sigmoid scores, top-k by value
    (ties to the lower expert id), weights renormalised to sum to one."""
    rng = np.random.default_rng(seed)
    logits = rng.standard_normal((num_tokens, num_experts), dtype=np.float32)
    scores = 1.0 / (1.0 + np.exp(-logits))
    order = np.argsort(-scores, axis=1, kind="stable")[:, :topk]
    picked = np.take_along_axis(scores, order, axis=1)
    weights = (picked / picked.sum(axis=1, keepdims=True)).astype(np.float32)
    return order.astype(np.int32), weights


def dirichlet_counts(total_rows: int, groups: int, seed: int, alpha: float = 0.5):
    rng = np.random.default_rng(seed)
    p = rng.dirichlet(np.full(groups, alpha))
    counts = rng.multinomial(total_rows, p).astype(np.int32)
    cu = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    return counts, cu
