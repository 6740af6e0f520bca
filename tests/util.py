"""Comparison rules of the parity tests.

  * cast / add / copy: bit-exact (compared as raw integer views);
  * row reductions: |a - b| <= 1e-3 * |b| + 1 fp16 ULP of b.  1e-3 relative is about one
    fp16 ULP (2^-10), and a different summation order can flip the final fp16 rounding by
    one ULP; softmax outputs reach the fp16 subnormal range where one ULP is far more than
    1e-3 relative.  The ULP term is stated, not hidden.  LayerNorm ends in `a * gamma + beta`,
    which cancels where the two terms are opposite: there the error is relative to the terms
    (|beta| ~ 0.1), not to the tiny result, so its tests add an absolute floor of 1e-6
    (1e-5 of the terms' magnitude);
  * GEMM / GEMV: |a - b| <= 1e-2 * |b| + 1e-2 * rms(b), against an fp32-accumulated reference.
"""
import os

import numpy as np

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(op):
    return np.load(os.path.join(GOLDEN_DIR, f"{op}.npz"))


def fused_operands(case, ins):
    """(x, w, bias, res1, res2) of a fused-matmul golden case from its input list."""
    x, w, rest = ins[0], ins[1], list(ins[2:])
    bias = rest.pop(0) if case.get("bias", True) else None
    rest += [None, None]
    return x, w, bias, rest[0], rest[1]


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view({1: np.uint8, 2: np.uint16, 4: np.uint32}[a.dtype.itemsize])


def assert_bit_exact(got, want, what=""):
    got, want = np.asarray(got), np.asarray(want)
    assert got.shape == want.shape and got.dtype == want.dtype, (what, got.shape, want.shape, got.dtype, want.dtype)
    bad = np.nonzero(bits(got).reshape(-1) != bits(want).reshape(-1))[0]
    assert bad.size == 0, f"{what}: {bad.size} of {got.size} elements differ, first at flat index {bad[0]}"


def fp16_ulp(x):
    """Spacing of fp16 numbers at |x| (subnormal spacing 2^-24 below 2^-14)."""
    ax = np.abs(np.asarray(x, np.float32))
    e = np.floor(np.log2(np.maximum(ax, 2.0 ** -14)))
    return np.exp2(e - 10).astype(np.float32)


def assert_reduction_close(got, want, what="", rel=1e-3, abs_floor=0.0):
    g = np.asarray(got, np.float32).reshape(-1)
    w = np.asarray(want, np.float32).reshape(-1)
    assert g.shape == w.shape, (what, g.shape, w.shape)
    assert np.isfinite(g).all(), f"{what}: non-finite values"
    tol = rel * np.abs(w) + fp16_ulp(w) + abs_floor
    err = np.abs(g - w)
    bad = np.nonzero(err > tol)[0]
    assert bad.size == 0, (f"{what}: {bad.size} of {g.size} outside 1e-3 rel + 1 fp16 ULP; worst "
                           f"got {g[bad[0]]} want {w[bad[0]]}")


def assert_matmul_close(got, want_f32, what="", rel=1e-2):
    g = np.asarray(got, np.float32).reshape(-1)
    w = np.asarray(want_f32, np.float32).reshape(-1)
    assert g.shape == w.shape, (what, g.shape, w.shape)
    assert np.isfinite(g).all(), f"{what}: non-finite values"
    rms = float(np.sqrt(np.mean(w.astype(np.float64) ** 2)))
    tol = rel * np.abs(w) + rel * rms
    err = np.abs(g - w)
    bad = np.nonzero(err > tol)[0]
    assert bad.size == 0, (f"{what}: {bad.size} of {g.size} outside 1e-2 rel (+1e-2 rms floor); worst "
                           f"got {g[bad[0]]} want {w[bad[0]]} rms {rms}")


def reference_tree():
    """Directory of a checkout of the reference (JackWeiw/dtas), or None: $DTAS_REFERENCE_TREE, else a
    directory named `reference` beside this repository.  Only CPU tests that re-derive fixtures use it;
    nothing that runs on a GPU box does."""
    cand = os.environ.get("DTAS_REFERENCE_TREE") or os.path.join(os.path.dirname(os.path.dirname(GOLDEN_DIR)), "..", "reference")
    cand = os.path.abspath(cand)
    return cand if os.path.isdir(os.path.join(cand, "python", "dtas")) else None


def load_ref_golden(key):
    return np.load(os.path.join(GOLDEN_DIR, f"ref_{key}.npz"))


def fp16_accumulation_bound(k, rms):
    """Error model of the reference's fp16 accumulator against exact summation: every one of the k
    updates rounds the running sum to fp16 (half an ULP at most, uniformly distributed), a random
    walk with sigma = ULP(rms) * sqrt(k / 12).  Eight sigma covers every element of the largest test
    (the worst of 51 200 outputs at k = 2560 sat at 4.7 sigma)."""
    return 8.0 * float(fp16_ulp(np.float32(rms))) * float(np.sqrt(k / 12.0))
