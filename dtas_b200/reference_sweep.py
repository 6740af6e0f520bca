"""The reference's own published sweeps, run on this library: same operators, dtypes, shapes and
row counts as the JSON files its profiling scripts committed (dolly-v2-3b, hidden size 2560):

    cast fp16 -> fp32, add fp16, copy fp16 on [1, n, 2560]   experiment/dtas_tuned/elementwise/*/profile_*.py
    layer norm + cast, fp32 [1, n, 2560] -> fp16             experiment/dtas_tuned/general_reduction/layernorm/profile_dlight.py:8-40
    softmax + cast, fp32 [1, 32, 400, m] -> fp16             experiment/dtas_tuned/general_reduction/softmax/profile_dlight.py:8-52
    NT matmul + bias, [n, K] x [N, K]^T                      experiment/testIR/GEMM/dlight.py:30-50
    GEMV 2560 x 10240                                        experiment/testIR/GEMV/m1n2560k10240/dlight_gemv.py:8-27

    python -m dtas_b200.reference_sweep [--out table.md]

Prints one markdown table: device time per call (CUDA-graph replay, operands rotated past L2),
achieved GB/s or TFLOP/s on the algorithmic bytes / flops, and the fraction of this GPU's measured
peak.  The GEMM accumulates in fp32 where the reference's schedule accumulates in fp16.
"""
import argparse
import sys

import torch

N_POINTS = [1, 17, 128, 256, 1025, 2049, 4096]
GEMM_N_POINTS = [16, 64, 255, 1024, 2048, 4096]
HIDDEN = 2560
SOFTMAX_ROWS = 32 * 400
SOFTMAX_LEN = [17, 128, 256, 1025, 2049, 4096]
GEMM_SHAPES = [(2560, 10240), (10240, 2560), (7680, 2560)]


def _sets(make, bytes_per_call):
    from .profiling import rotation_for
    return [make() for _ in range(rotation_for(bytes_per_call, max_copies=16))]


def _rand(shape, dtype, dev, scale=1.0):
    return (torch.randn(shape, device=dev, dtype=torch.float32) * scale).to(dtype)


def workloads(dev):
    """Yields (label, n, bytes, flops, list of operand sets, call(set))."""
    from . import ops
    f16, f32 = torch.float16, torch.float32
    for n in N_POINTS:
        e = n * HIDDEN
        yield ("cast fp16->fp32 [1,n,2560]", n, 6 * e, 0,
               _sets(lambda: (_rand((n, HIDDEN), f16, dev), torch.empty((n, HIDDEN), dtype=f32, device=dev)), 6 * e),
               lambda s: ops.cast(s[0], s[1]))
    for n in N_POINTS:
        e = n * HIDDEN
        yield ("add fp16 [1,n,2560]", n, 6 * e, 0,
               _sets(lambda: (_rand((n, HIDDEN), f16, dev), _rand((n, HIDDEN), f16, dev),
                              torch.empty((n, HIDDEN), dtype=f16, device=dev)), 6 * e),
               lambda s: ops.add(s[0], s[1], s[2]))
    for n in N_POINTS:
        e = n * HIDDEN
        yield ("copy fp16 [1,n,2560]", n, 4 * e, 0,
               _sets(lambda: (_rand((n, HIDDEN), f16, dev), torch.empty((n, HIDDEN), dtype=f16, device=dev)), 4 * e),
               lambda s: ops.copy(s[0], s[1]))
    gamma, beta = _rand((HIDDEN,), f32, dev), _rand((HIDDEN,), f32, dev)
    for n in N_POINTS:
        e = n * HIDDEN
        yield ("layer norm + cast fp32->fp16 [1,n,2560]", n, 6 * e, 0,
               _sets(lambda: (_rand((n, HIDDEN), f32, dev), torch.empty((n, HIDDEN), dtype=f16, device=dev)), 6 * e),
               lambda s: ops.layer_norm(s[0], gamma, beta, s[1]))
    for m in SOFTMAX_LEN:
        e = SOFTMAX_ROWS * m
        yield ("softmax + cast fp32->fp16 [1,32,400,m] (n = m)", m, 6 * e, 0,
               _sets(lambda: (_rand((SOFTMAX_ROWS, m), f32, dev), torch.empty((SOFTMAX_ROWS, m), dtype=f16, device=dev)), 6 * e),
               lambda s: ops.softmax(s[0], s[1]))
    for (N, K) in GEMM_SHAPES:
        bias = _rand((N,), f16, dev, 0.5)
        w_sets = _sets(lambda: _rand((N, K), f16, dev, 0.02), 2 * N * K)
        for n in GEMM_N_POINTS:
            x = _rand((n, K), f16, dev)
            y = torch.empty((n, N), dtype=f16, device=dev)
            yield (f"NT matmul + bias [n,{K}] x [{N},{K}]^T", n, 2 * (n * K + N * K + n * N), 2 * n * N * K,
                   [(x, w, y) for w in w_sets], lambda s, b=bias: ops.gemm_nt(s[0], s[1], s[2], bias=b))
    N, K = 2560, 10240
    x, y = _rand((1, K), f16, dev), torch.empty((1, N), dtype=f16, device=dev)
    yield ("GEMV [1,10240] x [2560,10240]^T", 1, 2 * N * K + 2 * K + 2 * N, 2 * N * K,
           [(x, w, y) for w in _sets(lambda: _rand((N, K), f16, dev, 0.02), 2 * N * K)],
           lambda s: ops.gemv(s[0], s[1], s[2]))


def main():
    from . import ops
    from .profiling import measured_peaks, time_op
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args()
    dev = torch.device("cuda", a.device)
    torch.cuda.set_device(dev)
    peaks, src = measured_peaks()
    lines = [f"Peaks ({src}): {peaks['hbm_gbs']:.0f} GB/s, {peaks['bf16_tflops']:.0f} TFLOP/s.", "",
             "| workload | n | us | GB/s | TFLOP/s | bound | fraction of peak |", "|---|---|---|---|---|---|---|"]
    for label, n, nbytes, flops, sets, call in workloads(dev):
        t = time_op(lambda i: call(sets[i % len(sets)]), warmup=3, number=3, min_repeat_ms=10.0, graph=True)
        ops.poll_status()
        us = t["mean_us"]
        t_hbm, t_tc = nbytes / peaks["hbm_gbs"] * 1e-3, flops / peaks["bf16_tflops"] * 1e-6      # us
        bound = "tensor" if t_tc > t_hbm else "hbm"
        lines.append(f"| {label} | {n} | {us:.2f} | {nbytes / us / 1e3:.0f} | {flops / us / 1e6:.1f} | {bound} | "
                     f"{max(t_hbm, t_tc) / us:.3f} |")
        del sets
    text = "\n".join(lines) + "\n"
    sys.stdout.write(text)
    if a.out:
        with open(a.out, "w") as f:
            f.write(text)


if __name__ == "__main__":
    main()
