"""Command-line launcher for one operator at one shape: a few launches on random data.

    python -m dtas_b200.run_op --op gemm --m 1024 --n 4096 --k 4096 --iters 3

Used for profiler captures (one small case per kernel) and as a quick check that the
library loads and launches on this machine.  Prints the kernel variant and the mean time.
"""
import argparse

import torch

from . import _abi, ops
from .profiling import algorithmic


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=["cast", "add", "copy", "rms_norm", "softmax", "gemv", "gemm"])
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--bn", type=int, default=0, help="gemm: force the tile width (0 = planner)")
    ap.add_argument("--split-k", type=int, default=0, help="gemm: force the split factor (0 = planner)")
    ap.add_argument("--tail", default="none", choices=["none", "bias", "gelu", "res2"],
                    help="gemm: what is fused behind the product (bias; bias + erf-GELU; bias + two residuals)")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    f16 = torch.float16
    m, n, k = a.m, a.n, a.k
    if a.op == "cast":
        x, y = torch.randn(m, n, device=dev), torch.empty(m, n, device=dev, dtype=f16)
        fn = lambda: ops.cast(x, y)  # noqa: E731
    elif a.op in ("add", "copy"):
        x = torch.randn(m, n, device=dev, dtype=f16)
        b, y = torch.randn_like(x), torch.empty_like(x)
        fn = (lambda: ops.add(x, b, y)) if a.op == "add" else (lambda: ops.copy(x, y))
    elif a.op in ("rms_norm", "softmax"):
        x = torch.randn(m, n, device=dev, dtype=f16)
        w, y = torch.ones(n, device=dev, dtype=f16), torch.empty_like(x)
        fn = (lambda: ops.rms_norm(x, w, y)) if a.op == "rms_norm" else (lambda: ops.softmax(x, y))
    elif a.op == "gemv":
        x, w = torch.randn(1, k, device=dev, dtype=f16), torch.randn(n, k, device=dev, dtype=f16) * 0.02
        y = torch.empty(1, n, device=dev, dtype=f16)
        fn = lambda: ops.gemv(x, w, y)  # noqa: E731
    else:
        _abi.check(_abi.lib().dtas_gemm_set_override(a.bn, a.split_k))
        x, w = torch.randn(m, k, device=dev, dtype=f16), torch.randn(n, k, device=dev, dtype=f16) * 0.02
        y = torch.empty(m, n, device=dev, dtype=f16)
        kw = {}
        if a.tail != "none":
            kw["bias"] = torch.randn(n, device=dev, dtype=f16)
        if a.tail == "gelu":
            kw["act"] = "gelu"
        if a.tail == "res2":
            kw["res1"], kw["res2"] = torch.randn(m, n, device=dev, dtype=f16), torch.randn(m, n, device=dev, dtype=f16)
        fn = lambda: ops.gemm_nt(x, w, y, **kw)  # noqa: E731
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ops.poll_status(0)
    us = 1e3 * e0.elapsed_time(e1) / a.iters
    alg = algorithmic(a.op, m, n, k if a.op in ("gemv", "gemm") else 0)
    print(f"{a.op} m={m} n={n} k={k}: {_abi.variant_of(a.op, m, n, k, 0)}  {us:.2f} us/launch  "
          f"{alg['bytes'] / us / 1e3:.0f} GB/s  {alg['flops'] / us / 1e6:.1f} TFLOP/s")


if __name__ == "__main__":
    main()
