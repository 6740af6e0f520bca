"""Timing harness: the protocol of the reference's measurements on CUDA events.

The reference times every candidate and every published number with TVM's
`time_evaluator(number=5, min_repeat_ms=50)` and reports the mean
(python/dtas/schedule/tir_base.py:208-210, experiment/dtas_tuned/elementwise/cast/profile_cast.py:9-22).
`time_op` does the same with CUDA events on the launching stream: warm-up, then batches of
launches bracketed by events until at least `min_repeat_ms` of device time and `number`
batches have run; it returns mean and min microseconds per launch.

To keep bandwidth figures honest the callable receives a rotating index, so the caller can
cycle through enough distinct buffers that the working set exceeds the 126 MB L2
(`rotation_for`); the reference's own >1 TiB/s points on a 936 GB/s card are L2 hits
(experiment/dtas_tuned/elementwise/cast/top10_256/bandwidth.json).
"""
import json
import os

import torch

L2_BYTES = 126 * 1024 * 1024
NOMINAL = {"hbm_gbs": 8000.0, "fp16_tflops": 2250.0}
FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def measured_peaks(root=None):
    """Reads MEASURED_PEAKS.json from the repository root (written per pod by the test
    driver); falls back to an earlier measurement of the same pool.  -> (dict, source)."""
    root = root or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"]))}, "measured"
    return dict(FALLBACK), "fallback"


def rotation_for(bytes_per_call, min_total=2 * L2_BYTES, max_copies=64):
    """How many distinct buffer sets a benchmark should cycle through so that consecutive
    launches cannot be served from L2."""
    if bytes_per_call <= 0:
        return 1
    n = -(-min_total // int(bytes_per_call))
    return int(max(1, min(max_copies, n)))


def time_op(fn, warmup=3, number=5, min_repeat_ms=50.0, batch=None, max_batches=200, stream=None,
            graph=False):
    """fn(i) launches the op once (i = running launch index).  Returns
    {"mean_us", "min_us", "launches", "batches"} measured with CUDA events on `stream`
    (default: the current torch stream, which is where dtas_b200.ops launches).

    graph=False times eager calls: what a Python caller sees, host overhead included when the
    kernel is shorter than the call path.  graph=True captures one batch of launches into a
    CUDA graph and replays it: device time of the kernels back to back, the figure to hold
    against a roofline.  The op calls allocate nothing and never synchronise, so they capture
    as they are (first-use set-up happens in the warm-up calls)."""
    stream = stream or torch.cuda.current_stream()
    it = 0
    for _ in range(max(1, warmup)):
        fn(it)
        it += 1
    stream.synchronize()
    if batch is None:
        # size a batch to roughly 2 ms so event overhead and launch gaps stay negligible
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(4):
            fn(it)
            it += 1
        e1.record(stream)
        e1.synchronize()
        per = max(e0.elapsed_time(e1) / 4.0, 1e-3)
        batch = int(max(1, min(400, round(2.0 / per))))
    replay = None
    if graph:
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(stream)
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                for j in range(batch):
                    fn(it + j)
        it += batch
        stream.wait_stream(side)
        replay = g.replay
        replay()
        stream.synchronize()
    times = []
    total_ms = 0.0
    while (len(times) < number or total_ms < min_repeat_ms) and len(times) < max_batches:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        if replay is not None:
            replay()
        else:
            for _ in range(batch):
                fn(it)
                it += 1
        e1.record(stream)
        e1.synchronize()
        ms = e0.elapsed_time(e1)
        times.append(ms / batch)
        total_ms += ms
    return {"mean_us": 1e3 * sum(times) / len(times), "min_us": 1e3 * min(times),
            "launches": batch * len(times), "batches": len(times), "mode": "graph" if graph else "eager"}


# Algorithmic bytes / flops per call of each operator (GB = 1e9 B).
def algorithmic(op, m, n, k=0):
    if op == "cast":            # fp32 in, fp16 out
        return {"bytes": 6 * m * n, "flops": 0}
    if op == "add":             # fp16: two reads, one write
        return {"bytes": 6 * m * n, "flops": 0}
    if op == "copy":
        return {"bytes": 4 * m * n, "flops": 0}
    if op == "rms_norm":
        return {"bytes": 4 * m * n + 2 * n, "flops": 0}
    if op == "softmax":
        return {"bytes": 4 * m * n, "flops": 0}
    if op == "gemv":
        return {"bytes": 2 * n * k + 2 * k + 2 * n, "flops": 2 * n * k}
    if op == "gemm":
        return {"bytes": 2 * (m * k + n * k + m * n), "flops": 2 * m * n * k}
    raise ValueError(op)
