"""Per-CTA timeline of a GEMM launch, from the trace build of the library.

    python -m dtas_b200.build --trace                      # lib/libdtas_b200_trace.so (-DDTAS_TRACE)
    python -m dtas_b200.trace_gemm --m 16 --n 4096 --k 4096 [--bn 1024 --split-k 4]

The single-CTA and swapped-operand GEMM kernels stamp their SM clock at a few milestones
(csrc/gemm_tcgen05.cu, DTAS_TRACE_AT).  The launch is replayed back to back from a CUDA graph with
W rotated beyond L2; the stamps of the last launch are read out with dtas_trace_read() and printed
relative to the moment the CTA passed the launch wait, as median / min / max over the CTAs, in
microseconds (the SM clock is taken as the maximum clock: check `nvidia-smi` if in doubt).
"""
import argparse
import ctypes
import os

MILESTONES = ["entry", "set-up done", "launch wait passed", "first TMA issued", "last TMA issued", "first operands in",
              "last MMA committed", "epilogue woke", "partial stored + fenced", "ticket known", "epilogue done",
              "all warps joined", "tensor memory freed"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, required=True)
    ap.add_argument("--n", type=int, required=True)
    ap.add_argument("--k", type=int, required=True)
    ap.add_argument("--bn", type=int, default=0, help="tile code as in dtas_gemm_set_override (0 = dispatch)")
    ap.add_argument("--split-k", type=int, default=0)
    ap.add_argument("--sm-ghz", type=float, default=1.965)
    a = ap.parse_args()

    from .build import TRACE_LIB_PATH
    if not os.path.exists(TRACE_LIB_PATH):
        raise SystemExit(f"{TRACE_LIB_PATH} is missing: python -m dtas_b200.build --trace")
    os.environ["DTAS_B200_LIB"] = TRACE_LIB_PATH
    import numpy as np
    import torch
    from . import _abi, ops
    from .profiling import algorithmic, rotation_for, time_op

    lib = _abi.lib()
    lib.dtas_trace_read.restype = ctypes.c_int
    lib.dtas_trace_read.argtypes = [ctypes.c_void_p]
    dev = torch.device("cuda", torch.cuda.current_device())
    copies = rotation_for(algorithmic("gemm", a.m, a.n, a.k)["bytes"], max_copies=16)
    f16 = dict(dtype=torch.float16, device=dev)
    x, y = torch.randn(a.m, a.k, **f16), torch.empty(a.m, a.n, **f16)
    ws = [torch.randn(a.n, a.k, **f16) * 0.02 for _ in range(copies)]
    _abi.check(lib.dtas_gemm_set_override(a.bn, a.split_k))
    try:
        variant = _abi.variant_of("gemm", a.m, a.n, a.k)
        if "2cta" in variant or "simt" in variant:
            raise SystemExit(f"{variant}: only the single-CTA and swapped-operand kernels are instrumented")
        t = time_op(lambda i: ops.gemm_nt(x, ws[i % copies], y), graph=True, min_repeat_ms=10.0)
        torch.cuda.synchronize()
    finally:
        lib.dtas_gemm_set_override(0, 0)
    buf = np.zeros((1024, 16), dtype=np.uint64)
    _abi.check(lib.dtas_trace_read(buf.ctypes.data))
    tr = buf.astype(np.int64)
    live = tr[:, 15] > tr[:, 15].max() - int(t["mean_us"] * 1000 * 0.8)     # CTAs of the last launch (global timer at exit)
    c = tr[live]
    print(f"m={a.m} n={a.n} k={a.k} {variant}: {t['mean_us']:.2f} us per launch, {int(live.sum())} CTAs")
    print(f"  entry skew {np.ptp(c[:, 14]) / 1e3:.2f} us, exit skew {np.ptp(c[:, 15]) / 1e3:.2f} us (global timer)")
    rel = (c[:, :13] - c[:, 2:3]) / (a.sm_ghz * 1e3)
    shared = "splitk1" not in variant
    for i, name in enumerate(MILESTONES):
        if i in (8, 9) and not shared:
            continue
        col = rel[:, i][c[:, i] > 0]
        if len(col):
            print(f"  {i:2d} {name:26s} median {np.median(col):7.2f}   min {col.min():7.2f}   max {col.max():7.2f}")
    if shared:
        red = (c[:, 10] - c[:, 9]) / (a.sm_ghz * 1e3)
        last = red > 0.4
        if last.any():
            print(f"  last arrivers ({int(last.sum())} CTAs): read-back and store {np.median(red[last]):.2f} us (median), "
                  f"{red[last].max():.2f} max")


if __name__ == "__main__":
    main()
