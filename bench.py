"""Benchmark of the dtas_b200 hot path: the dynamic-m operator sweep.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One STEP launches every point of the five measured configurations once (cast fp32->fp16 at
m in {1,17,128,4096}; fp16 add and copy on [m,11008] at m in {1,7,64,512,8192}; RMSNorm and
softmax on [m,4096] at m in {1,33,256,4096}; the four Llama-2-7B GEMVs; the four GEMM shapes
at m in {16,64,255,1024,4096,8192}): 50 kernels of this library, operands resident in HBM,
synthetic seeded data.  The timed region is exactly K steps between two barriers +
synchronisations, timed with CUDA events on the launching stream, max over ranks.

    value = 100 * (time the step would take at the roofline of ONE B200) / (measured time)

where the roofline time of a point is max(algorithmic bytes / measured HBM bandwidth,
flops / measured dense 16-bit tensor throughput) with the peaks of MEASURED_PEAKS.json.
With N GPUs the same sweep is sharded (GEMM / GEMV by output columns, the other ops by rows,
no collective on the data path; "scaling": "strong") and the value is still relative to one
GPU's roofline, so value(N) / value(1) is the speed-up.

Also reported: per-point device times from CUDA-graph replay ("points", with the fraction of the
measured and of the data-sheet peaks), the roofline of the dominant kernel, an end-to-end figure
through the public API with host buffers ("e2e"), the CPU baseline, SM clocks during the timed
region, the number of kernels launched and, with N > 1, what gathering a column-sharded result
onto every rank adds ("gathered_points": kernel alone against kernel + one NCCL all-gather).

`--impl reference` times the reference workload PrimFuncs on the host CPU instead (built by
TVM for target "c" when that runtime is available on the box, else the C port under oracle/).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CAST_M = [1, 17, 128, 4096]
EW_M = [1, 7, 64, 512, 8192]
ROW_M = [1, 33, 256, 4096]
GEMV_SHAPES = [(4096, 4096), (11008, 4096), (4096, 11008), (32000, 4096)]
GEMM_SHAPES = [(12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008)]
GEMM_M = [16, 64, 255, 1024, 4096, 8192]
METRIC = "% of roofline (HBM GB/s or fp16 TFLOP/s) across dynamic m"
UNIT = "% of one B200's roofline over the sweep (time-weighted, measured peaks)"
WORKLOAD = ("dynamic-m operator sweep: cast f32->f16 [m,4096]; add+copy f16 [m,11008]; rms_norm+softmax f16 "
            "[m,4096]; gemv f16 x4 Llama-2-7B shapes; gemm f16 NT x4 shapes, m in {16,64,255,1024,4096,8192}")


def sweep_points():
    """(op, m, n, k) of every kernel launch of one step."""
    pts = [("cast", m, 4096, 0) for m in CAST_M]
    for m in EW_M:
        pts += [("add", m, 11008, 0), ("copy", m, 11008, 0)]
    for m in ROW_M:
        pts += [("rms_norm", m, 4096, 0), ("softmax", m, 4096, 0)]
    pts += [("gemv", 1, n, k) for (n, k) in GEMV_SHAPES]
    for (n, k) in GEMM_SHAPES:
        pts += [("gemm", m, n, k) for m in GEMM_M]
    return pts


def bench_config(peaks, peak_src):
    """The `config` object of the JSON line: the same in both arms, so their figures can be divided."""
    return {"workload": WORKLOAD,
            "l2": "inputs larger than L2: one step streams about 4 GB of distinct operands, so no buffer "
                  "survives in the 126 MB L2 until its next use",
            "peaks": {**peaks, "source": peak_src}}


def roofline_ns(op, m, n, k, peaks):
    from dtas_b200.profiling import algorithmic
    a = algorithmic(op, m, n, k)
    t_hbm = a["bytes"] / peaks["hbm_gbs"]                     # bytes / (GB/s) = ns
    t_tc = a["flops"] / (peaks["bf16_tflops"] * 1e3)          # flop / (TFLOP/s) = ps -> /1e3 = ns
    return max(t_hbm, t_tc), ("tensor" if t_tc > t_hbm else "hbm")


def nominal_ns(op, m, n, k):
    """The same bound at the data-sheet peaks (8 TB/s, 2.25 PFLOP/s dense fp16)."""
    from dtas_b200.profiling import NOMINAL
    return roofline_ns(op, m, n, k, {"hbm_gbs": NOMINAL["hbm_gbs"], "bf16_tflops": NOMINAL["fp16_tflops"]})[0]


def shard(total, rank, world):
    """Contiguous split with the remainder on the low ranks -> (start, count)."""
    base, rem = divmod(total, world)
    count = base + (1 if rank < rem else 0)
    start = rank * base + min(rank, rem)
    return start, count


# -----------------------------------------------------------------------------------------
# clocks
# -----------------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, reasons, mx = [], set(), None
        try:
            with open(self.path) as f:
                for line in f:
                    c = [x.strip() for x in line.split(",")]
                    if len(c) < 9 or not c[1].isdigit():
                        continue
                    sm.append(int(c[1]))
                    mx = int(c[2]) if c[2].isdigit() else mx
                    for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=mx, reasons=sorted(reasons), samples=len(sm))
        return out


# -----------------------------------------------------------------------------------------
# the GPU arm
# -----------------------------------------------------------------------------------------
class Sweep:
    """Device-resident operands of this rank's share of the sweep, and the launch list."""

    def __init__(self, rank, world, dev):
        import torch
        from dtas_b200 import Engine, arch, ops, set_log_level
        set_log_level(0)
        from dtas_b200.workloads import llama2_7b_specs
        self.torch, self.rank, self.world, self.dev = torch, rank, world, dev
        self.rt = Engine(1, True, None).tune_module(llama2_7b_specs(), arch=arch.B200(dev.index), range_div_factor=256)
        g = torch.Generator(device=dev).manual_seed(1234 + rank)

        def randn(shape, dtype, scale=1.0):
            t = torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
            return (t * scale).to(dtype) if scale != 1.0 else t.to(dtype)

        f16, f32 = torch.float16, torch.float32
        self.calls = []      # (point, callable(i)): i picks one of the point's rotating buffer sets
        self.h2d_bytes = 0   # per step, for the e2e arm (activations only; weights stay resident)
        self.d2h_bytes = 0
        self.e2e = []        # (host inputs, device inputs, device output, host output)
        self.launch_points = []

        def add_call(point, fn, ins, out, pre=None):
            self.calls.append((point, fn))
            self.launch_points.append(point)
            self.e2e.append((ins, out, pre))

        for m in CAST_M:
            _, rows = shard(m, rank, world)
            if rows == 0:
                continue
            x, y = randn((rows, 4096), f32), torch.empty((rows, 4096), dtype=f16, device=dev)
            add_call(("cast", m, 4096, 0), (lambda x=x, y=y: self.rt["cast"](x, y)), [x], y)
        for m in EW_M:
            _, rows = shard(m, rank, world)
            if rows == 0:
                continue
            a, b = randn((rows, 11008), f16), randn((rows, 11008), f16)
            c, d = torch.empty_like(a), torch.empty_like(a)
            add_call(("add", m, 11008, 0), (lambda a=a, b=b, c=c: self.rt["add"](a, b, c)), [a, b], c)
            add_call(("copy", m, 11008, 0), (lambda a=a, d=d: self.rt["copy"](a, d)), [a], d)
        w_norm = randn((4096,), f16, 0.1) + 1
        for m in ROW_M:
            _, rows = shard(m, rank, world)
            if rows == 0:
                continue
            x = randn((rows, 4096), f16)
            y, z = torch.empty_like(x), torch.empty_like(x)
            add_call(("rms_norm", m, 4096, 0), (lambda x=x, y=y: self.rt["rms_norm"](x, w_norm, y)), [x], y)
            add_call(("softmax", m, 4096, 0), (lambda x=x, z=z: self.rt["softmax"](x, z)), [x], z)
        for (n, k) in GEMV_SHAPES:
            _, cols = shard(n, rank, world)
            w = randn((cols, k), f16, 0.02)
            x, y = randn((1, k), f16), torch.empty((1, cols), dtype=f16, device=dev)
            name = f"gemv_n{n}_k{k}"
            fn = (lambda x=x, w=w, y=y, name=name: self.rt[name](x, w, y)) if world == 1 else \
                 (lambda x=x, w=w, y=y: ops.gemv(x, w, y))
            add_call(("gemv", 1, n, k), fn, [x], y)
        for (n, k) in GEMM_SHAPES:
            _, cols = shard(n, rank, world)
            w = randn((cols, k), f16, 0.02)
            name = f"gemm_n{n}_k{k}"
            for m in GEMM_M:
                y = torch.empty((m, cols), dtype=f16, device=dev)
                if world == 1:
                    x = randn((m, k), f16)
                    add_call(("gemm", m, n, k), (lambda x=x, w=w, y=y, name=name: self.rt[name](x, w, y)), [x], y)
                    continue
                # X is replicated for the kernels.  End to end every rank uploads only its share of the
                # rows and the ranks exchange them over NVLink (one NCCL all-gather in place), instead of
                # every rank pulling the whole X through the host's PCIe.
                per = -(-m // world)
                x_pad = randn((world * per, k), f16)
                x, mine = x_pad[:m], x_pad[rank * per:(rank + 1) * per]

                def gather_x(x_pad=x_pad, mine=mine):
                    import torch.distributed as dist
                    dist.all_gather_into_tensor(x_pad.view(-1), mine.reshape(-1))

                add_call(("gemm", m, n, k), (lambda x=x, w=w, y=y: ops.gemm_nt(x, w, y)), [mine], y, pre=gather_x)
        for ins, out, _ in self.e2e:
            self.h2d_bytes += sum(t.numel() * t.element_size() for t in ins)
            self.d2h_bytes += out.numel() * out.element_size()

    def step(self):
        for _, fn in self.calls:
            fn()


def point_runner(op, m, n, k, dev):
    """-> (fn(i), copies): launches one point on operand set i % copies."""
    import torch
    from dtas_b200 import ops
    from dtas_b200.profiling import algorithmic, rotation_for
    f16 = torch.float16
    copies = rotation_for(algorithmic(op, m, n, k)["bytes"], max_copies=16)

    def rnd(shape, dtype=f16, scale=1.0):
        return (torch.randn(shape, device=dev, dtype=torch.float32) * scale).to(dtype)

    if op == "cast":
        xs = [rnd((m, n), torch.float32) for _ in range(copies)]
        ys = [torch.empty((m, n), dtype=f16, device=dev) for _ in range(copies)]
        return (lambda i: ops.cast(xs[i % copies], ys[i % copies])), copies
    if op in ("add", "copy"):
        xs = [rnd((m, n)) for _ in range(copies)]
        bs = [rnd((m, n)) for _ in range(copies)] if op == "add" else None
        ys = [torch.empty((m, n), dtype=f16, device=dev) for _ in range(copies)]
        if op == "add":
            return (lambda i: ops.add(xs[i % copies], bs[i % copies], ys[i % copies])), copies
        return (lambda i: ops.copy(xs[i % copies], ys[i % copies])), copies
    if op in ("rms_norm", "softmax"):
        xs = [rnd((m, n)) for _ in range(copies)]
        ys = [torch.empty((m, n), dtype=f16, device=dev) for _ in range(copies)]
        w = rnd((n,), scale=0.1) + 1
        if op == "rms_norm":
            return (lambda i: ops.rms_norm(xs[i % copies], w, ys[i % copies])), copies
        return (lambda i: ops.softmax(xs[i % copies], ys[i % copies])), copies
    ws = [rnd((n, k), scale=0.02) for _ in range(copies)]
    if op == "gemv":
        x, y = rnd((1, k)), torch.empty((1, n), dtype=f16, device=dev)
        return (lambda i: ops.gemv(x, ws[i % copies], y)), copies
    x, y = rnd((m, k)), torch.empty((m, n), dtype=f16, device=dev)
    return (lambda i: ops.gemm_nt(x, ws[i % copies], y)), copies


POINT_IDLE_S = 0.2   # idle time before each per-point measurement


def fused_points(dev, peaks):
    """The fused matmul forms of the reference's model workloads at their own sizes (dolly-v2-3b:
    hidden 2560, FFN 10240): device time of the fused call, and of the same result from the plain
    GEMM followed by separate add kernels.  Not part of the step; reported beside it."""
    import torch
    from dtas_b200 import ops
    from dtas_b200.profiling import rotation_for, time_op
    f16 = dict(dtype=torch.float16, device=dev)
    out = []
    for m in (16, 1024, 4096):
        for label, n, k, n_res, act in (("gemm+bias+res+res", 2560, 2560, 2, None), ("gemm+bias+gelu", 10240, 2560, 0, "gelu")):
            nbytes = 2 * (m * k + n * k + m * n) + 2 * n + 2 * n_res * m * n
            flops = 2 * m * n * k
            copies = rotation_for(nbytes, max_copies=16)
            ws = [torch.randn(n, k, **f16) * 0.02 for _ in range(copies)]
            x, b, y, tmp = torch.randn(m, k, **f16), torch.randn(n, **f16), torch.empty(m, n, **f16), torch.empty(m, n, **f16)
            res = [torch.randn(m, n, **f16) for _ in range(n_res)] + [None, None]

            def fused(i):
                ops.gemm_nt(x, ws[i % copies], y, bias=b, res1=res[0], res2=res[1], act=act)

            def unfused(i):
                ops.gemm_nt(x, ws[i % copies], y, bias=b)
                if n_res:
                    ops.add(res[0], y, tmp)
                    ops.add(tmp, res[1], y)

            torch.cuda.synchronize()
            time.sleep(POINT_IDLE_S)
            tf = time_op(fused, warmup=3, number=3, min_repeat_ms=10.0, graph=True)["mean_us"]
            tu = time_op(unfused, warmup=3, number=3, min_repeat_ms=10.0, graph=True)["mean_us"]
            ideal_us = max(nbytes / (peaks["hbm_gbs"] * 1e3), flops / (peaks["bf16_tflops"] * 1e6))
            out.append({"op": label, "m": m, "n": n, "k": k, "us": round(tf, 2),
                        "us_unfused" if n_res else "us_plain_gemm": round(tu, 2), "frac": round(ideal_us / tf, 3)})
            del ws
    torch.cuda.empty_cache()
    return out


GATHER_POINTS = [("gemm", 8192, 22016, 4096), ("gemm", 64, 4096, 4096), ("gemv", 1, 32000, 4096)]


def gather_points(rank, world, dev, barrier, multicast=True, engines=("kernel", "copy", "epilogue")):
    """N > 1 only: what a caller pays who needs the whole Y on every rank.  Per point the kernel
    alone (this rank's column slab, written into its slot of the [g, m, N/g] buffer) and the
    kernel followed by one NCCL all-gather of that buffer, and the same result by pushing row
    blocks into the peers' buffers behind the kernel (this library's push kernel, or one
    cudaMemcpyAsync per peer), or by the GEMM whose epilogue stores every tile to the peers as well
    (dtas_gemm_nt_scatter + one barrier), all timed with CUDA events on the launching stream over a batch of
    eager calls, max over ranks.  Weights rotate through enough
    copies that a shard is not served from L2."""
    import torch
    import torch.distributed as dist
    from dtas_b200.dist import ColumnShardedLinear, PeerGatherBuffer
    from dtas_b200.profiling import rotation_for
    f16 = torch.float16
    out = []
    for (op, m, n, k) in GATHER_POINTS:
        if n % world:
            continue
        n_local = n // world
        copies = min(8, rotation_for(2 * n_local * k))
        gen = torch.Generator(device=dev).manual_seed(77 + rank)
        x = torch.randn((m, k), generator=gen, device=dev, dtype=torch.float32).to(f16)
        lins = [ColumnShardedLinear((torch.randn((n_local, k), generator=gen, device=dev, dtype=torch.float32) * 0.02).to(f16),
                                    n, rank=rank, world=world, already_sharded=True) for _ in range(copies)]
        buf = lins[0].gather_buffer(m, f16, dev)
        reps = 20 if m >= 1024 else 100

        def timed(fn):
            for i in range(3):
                fn(i)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(reps):
                fn(i)
            e1.record()
            e1.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) * 1e3 / reps], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        if engines != ("multicast",):
            local_us = timed(lambda i: lins[i % copies].forward_local(x, out=buf[rank]))
            gathered_us = timed(lambda i: lins[i % copies].forward_gathered(x, buf=buf))
        pushed = {}
        for engine in engines:
            pushed[engine] = None
            if engine in ("epilogue", "multicast") and m < 129:
                continue                       # the GEMM that stores to the peers itself needs 129 rows
            pbuf = PeerGatherBuffer(world, m, n_local, f16, dev, engine="epilogue" if engine == "multicast" else engine)
            if engine == "multicast":
                if not pbuf.has_multicast():   # no multicast mapping of symmetric memory on this system
                    del pbuf
                    continue
                pbuf.engine = "multicast"
            pushed[engine] = timed(lambda i: lins[i % copies].forward_pushed(x, pbuf, min_push_bytes=0))
            if engine in ("epilogue", "multicast"):
                # what arrived in the peers' slots of this rank's buffer is what an all-gather delivers
                want = lins[0].forward_gathered(x).clone()
                got = lins[0].forward_pushed(x, pbuf, min_push_bytes=0)
                torch.cuda.synchronize()
                flag = torch.tensor([int(torch.equal(got, want))], device=dev, dtype=torch.int32)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                pushed[engine + "_equals_all_gather"] = bool(flag.item())
            del pbuf
        if engines == ("multicast",):
            return pushed
        out.append({"op": op, "m": m, "n": n, "k": k, "kernel_us": round(local_us, 2),
                    "kernel_plus_all_gather_us": round(gathered_us, 2),
                    "kernel_plus_peer_push_us": round(pushed["kernel"], 2),
                    "kernel_plus_copy_engine_push_us": round(pushed["copy"], 2),
                    "gemm_storing_to_peers_us": None if pushed["epilogue"] is None else round(pushed["epilogue"], 2),
                    "gemm_storing_to_peers_equals_all_gather": pushed.get("epilogue_equals_all_gather"),
                    "gemm_storing_through_multicast_us": None, "gemm_storing_through_multicast_equals_all_gather": None,
                    "gather_bytes_per_rank": 2 * m * n_local, "mode": "eager calls, max over ranks"})
        del lins, buf, x
        torch.cuda.empty_cache()
    if engines != ("multicast",) and multicast and out and GATHER_POINTS[0][1] >= 129 and GATHER_POINTS[0][2] % world == 0:
        # the route through the switch's multicast last, on the first point only, and on its own: whatever
        # happens to it, the figures above stand
        try:
            mc = gather_points(rank, world, dev, barrier, engines=("multicast",))
            if mc.get("multicast") is not None:
                out[0]["gemm_storing_through_multicast_us"] = round(mc["multicast"], 2)
                out[0]["gemm_storing_through_multicast_equals_all_gather"] = mc.get("multicast_equals_all_gather")
        except Exception as e:  # noqa: BLE001
            out[0]["gemm_storing_through_multicast_error"] = f"{type(e).__name__}: {e}"[:200]
    return out


def multi_gpu_check(rank, world, dev):
    """N > 1: one small GEMM and one GEMV through the sharded path, gathered onto every rank, checked
    against an fp32 CPU product (1e-2 relative + 1e-2 rms) and, bit for bit, against the slab the rank's
    own kernel wrote without any gather.  Every rank checks; the line carries the AND over ranks."""
    import torch
    import torch.distributed as dist
    from dtas_b200.dist import ColumnShardedLinear
    from dtas_b200.reference import seeded_normal
    out = {}
    for name, m, n, k in (("gemm", 64, 4096, 1024), ("gemv", 1, 4096, 4096)):
        if n % world:
            continue
        x = seeded_normal((m, k), 4242, "float16")
        w = seeded_normal((n, k), 4243, "float16", scale=0.02)
        lin = ColumnShardedLinear(w.to(dev), n, rank=rank, world=world)
        xd = x.to(dev)
        local = lin.forward_local(xd).clone()
        full = ColumnShardedLinear.as_row_major(lin.forward_gathered(xd)).float().cpu()
        ref = x.float() @ w.float().T
        rms = float(ref.double().pow(2).mean().sqrt())
        excess = float(((full - ref).abs() - (1e-2 * ref.abs() + 1e-2 * rms)).max())
        same = bool(torch.equal(full[:, lin.col_start:lin.col_start + lin.n_local], local.float().cpu()))
        flags = torch.tensor([int(excess <= 0), int(same)], device=dev, dtype=torch.int32)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        out[name] = {"m": m, "n": n, "k": k, "within_1e-2_of_fp32_on_every_rank": bool(flags[0].item()),
                     "gathered_equals_ungathered_bits_on_every_rank": bool(flags[1].item()),
                     "worst_excess_rank0": round(excess, 6)}
    return out


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from dtas_b200 import _abi
    from dtas_b200.profiling import measured_peaks, time_op

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks, peak_src = measured_peaks(ROOT)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    mg_check = multi_gpu_check(rank, world, dev) if world > 1 else None
    sweep = Sweep(rank, world, dev)
    points = sweep_points()
    ideal_ns = sum(roofline_ns(*p, peaks)[0] for p in points)

    # ---- timed region: W warm-up steps, then exactly K steps ------------------------------
    for _ in range(max(3, args.warmup)):
        sweep.step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    launches0 = _abi.launch_count()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        sweep.step()
    e1.record()
    barrier()
    elapsed_ms = e0.elapsed_time(e1)
    launches = _abi.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    _abi.check(_abi.lib().dtas_poll_status(local))
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
        lt = torch.tensor([launches], device=dev, dtype=torch.int64)
        dist.all_reduce(lt, op=dist.ReduceOp.SUM)
        launches = int(lt.item())
    ms_per_step = elapsed_ms / args.steps
    value = 100.0 * (ideal_ns * 1e-6) / ms_per_step
    value_nominal = 100.0 * (sum(nominal_ns(*p) for p in points) * 1e-6) / ms_per_step

    # ---- end to end through the public API with host buffers ------------------------------
    pinned_in = [[torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for t in ins] for ins, _, _ in sweep.e2e]
    pinned_out = [torch.empty(out.shape, dtype=out.dtype, pin_memory=True) for _, out, _ in sweep.e2e]

    # Copies in, kernels and copies out run on three streams chained by events, so PCIe works in
    # both directions while the kernels run; per operator the order in -> kernel -> out is kept,
    # and a buffer is not overwritten before its previous reader has finished.
    s_in, s_out, s_main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
    n_ops = len(sweep.calls)
    ev_in = [torch.cuda.Event() for _ in range(n_ops)]
    ev_done = [torch.cuda.Event() for _ in range(n_ops)]
    ev_out = [torch.cuda.Event() for _ in range(n_ops)]
    primed = [False]

    def e2e_step():
        for i, ((ins, out, pre), hin, hout, (_, fn)) in enumerate(zip(sweep.e2e, pinned_in, pinned_out, sweep.calls)):
            with torch.cuda.stream(s_in):
                if primed[0]:
                    s_in.wait_event(ev_done[i])        # last step's kernel has read these inputs
                for d, h in zip(ins, hin):
                    d.copy_(h, non_blocking=True)
                ev_in[i].record(s_in)
            s_main.wait_event(ev_in[i])
            if primed[0]:
                s_main.wait_event(ev_out[i])           # last step's result has left the output buffer
            if pre is not None:
                pre()                                  # N > 1: the ranks exchange their rows of X over NVLink
            fn()
            ev_done[i].record(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[i])
                hout.copy_(out, non_blocking=True)
                ev_out[i].record(s_out)
        primed[0] = True

    e2e_steps = max(1, min(args.steps, 3))
    e2e_step()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    s_main.wait_stream(s_out)      # the last results have reached the host before the clock stops
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
        hb = torch.tensor([sweep.h2d_bytes, sweep.d2h_bytes], device=dev, dtype=torch.int64)
        dist.all_reduce(hb, op=dist.ReduceOp.SUM)
        h2d, d2h = int(hb[0].item()), int(hb[1].item())
    else:
        h2d, d2h = sweep.h2d_bytes, sweep.d2h_bytes
    del pinned_in, pinned_out

    # ---- per-point device times (CUDA-graph replay) on this rank's shard ---------------------
    # Each point cycles through enough distinct operand sets that consecutive launches cannot
    # be served from the 126 MB L2 (rotation_for).
    per_point, dominant = [], None
    if not args.no_points:
        from dtas_b200.profiling import algorithmic
        for (op, m, n, k) in points:
            n_local = shard(n, rank, world)[1] if op in ("gemv", "gemm") else n
            m_local = m if op in ("gemv", "gemm") else shard(m, rank, world)[1]
            if m_local == 0 or n_local == 0:
                continue
            fn, copies = point_runner(op, m_local, n_local, k, dev)
            # A point is timed on its own: after the m = 8192 GEMMs the SM clock stays under the power
            # cap for a while, which reads as +10-25 % on the small points that follow them.
            torch.cuda.synchronize()
            time.sleep(POINT_IDLE_S)
            # the reference's protocol: time_evaluator(number=5, min_repeat_ms=50)
            # (python/dtas/schedule/tir_base.py:208-210)
            t = time_op(fn, warmup=3, number=5, min_repeat_ms=50.0, graph=True)
            del fn
            ns, bound = roofline_ns(op, m_local, n_local, k, peaks)
            a = algorithmic(op, m_local, n_local, k)
            per_point.append({"op": op, "m": m, "n": n, "k": k, "us": round(t["mean_us"], 2), "bound": bound,
                              "frac": round(ns * 1e-3 / t["mean_us"], 3),
                              "frac_nominal": round(nominal_ns(op, m_local, n_local, k) * 1e-3 / t["mean_us"], 3),
                              "gbs": round(a["bytes"] / t["mean_us"] / 1e3, 1),
                              "tflops": round(a["flops"] / t["mean_us"] / 1e6, 1), "copies": copies,
                              "variant": _abi.variant_of(op, m_local, n_local, k, local)})
            if op == "gemm" and (dominant is None or t["mean_us"] > dominant[1]["mean_us"]):
                dominant = ((op, m_local, n_local, k), t)
        torch.cuda.empty_cache()
    fused = fused_points(dev, peaks) if (per_point and world == 1) else None
    gathered = None
    if world > 1 and not args.no_points:
        try:
            gathered = gather_points(rank, world, dev, barrier)
        except Exception as e:  # noqa: BLE001 - the extras are reported, never allowed to cost the bench line
            gathered = [{"error": f"{type(e).__name__}: {e}"[:300]}]
    roofline = None
    if dominant is not None:
        (op, m, n, k), t = dominant
        achieved = algorithmic(op, m, n, k)["flops"] / t["mean_us"] / 1e6
        roofline = {"bound": "tensor", "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": round(achieved / peaks["bf16_tflops"], 3),
                    "traffic": GEMM_NCU_TRAFFIC_BYTES if (m, n, k) == (8192, 22016, 4096) else None,
                    "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel at this "
                                      "shape from a separate ncu capture, not measured in this run; null when sharded",
                    "algorithmic_bytes": algorithmic(op, m, n, k)["bytes"],
                    "kernel": f"{_abi.variant_of(op, m, n, k, local)} m={m} n={n} k={k}", "peak_source": f"{peak_src}, burst",
                    "frac_of_sustained": round(achieved / peaks["bf16_tflops_sustained"], 3),
                    "launch_us": round(t["mean_us"], 1)}

    cpu = cpu_baseline(sample_seconds=args.cpu_seconds) if (rank == 0 and world == 1 and not args.no_cpu) else None

    if rank == 0:
        mean_frac = round(sum(p["frac"] for p in per_point) / len(per_point), 3) if per_point else None
        # how many points meet the targets: 0.80 of the HBM roofline, 0.65 of the tensor peak (GEMM, m >= 1024)
        summary = None
        if per_point:
            def target(p):
                return 0.65 if p["bound"] == "tensor" else 0.80
            summary = {"points": len(per_point), "mean_frac": mean_frac,
                       "meeting_target_measured_peaks": sum(1 for p in per_point if p["frac"] >= target(p)),
                       "meeting_target_nominal_peaks": sum(1 for p in per_point if p["frac_nominal"] >= target(p)),
                       "min_frac": min(p["frac"] for p in per_point),
                       "timing": "CUDA-graph replay, number=5, min_repeat_ms=50 per point, operand sets rotated beyond L2"}
            if roofline is not None:
                roofline["points_summary"] = summary
        line = {
            "metric": METRIC,
            "value": round(value, 2), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16 (fp32 accumulate)",
            "data": "synthetic (seeded normal; weights N(0,0.02))",
            "config": bench_config(peaks, peak_src),
            "kernels_per_step": len(points),
            "sharding": "single GPU" if world == 1 else f"gemm/gemv by output columns, other ops by rows, {world} ranks, no collective",
            "roofline": roofline,
            "cpu_baseline": cpu,
            "e2e": {"value": round(100.0 * (ideal_ns * 1e-6) / e2e_ms, 3), "unit": UNIT,
                    "ms_per_step": round(e2e_ms, 3), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "note": "RuntimeModule calls on pinned host buffers: activations copied in and results copied out "
                            "every step on copy streams chained to the kernels by events; weights stay resident"
                            + ("" if world == 1 else "; each rank uploads its share of the rows of every GEMM's X and the "
                               "ranks all-gather them over NVLink; each rank downloads its own column slab")},
            "gpu_launches": launches,
            "clocks": clocks,
            "value_vs_nominal_peaks": round(value_nominal, 2),
            "mean_point_frac": mean_frac,
            "points_summary": summary,
            "multi_gpu_check": mg_check,
            "points": per_point,
            "fused_points": fused,
            "gathered_points": gathered,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant GEMM
# (m=8192, n=22016, k=4096, two-CTA kernel), from an ncu capture of that launch
# (865.4 MB read + 344.5 MB written); a profile figure, carried here so the line is self-contained.
GEMM_NCU_TRAFFIC_BYTES = 1209894144


# -----------------------------------------------------------------------------------------
# CPU arms
# -----------------------------------------------------------------------------------------
def _cpu_point_time(op, m, n, k, backend, budget_s):
    """Seconds the CPU implementation needs for one full point, measured on a bounded sample
    (a slab of rows) and scaled linearly to the full row count.  -> (seconds, sample rows)."""
    import numpy as np
    import oracle
    from dtas_b200.reference import seeded_normal
    use_tvm = backend == "reference"
    if use_tvm:
        from oracle import ref_runner

    def timed(fn, reps=1):
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        return (time.perf_counter() - t0) / reps

    rows = m
    if op in ("cast", "add", "copy", "rms_norm", "softmax"):
        rows = min(m, 256)
        x32 = seeded_normal((1, rows, n), 1, "float32").numpy()
        x16 = x32.astype(np.float16)
        if op == "cast":
            fn = ref_runner.prepare("cast", x32, np.zeros((1, rows, n), np.float16)) if use_tvm else (lambda: oracle.cast(x32, np.float16))
        elif op == "add":
            fn = ref_runner.prepare("add", x16, x16, np.zeros_like(x16)) if use_tvm else (lambda: oracle.add(x16, x16))
        elif op == "copy":
            fn = ref_runner.prepare("copy", x16, np.zeros_like(x16)) if use_tvm else (lambda: oracle.copy(x16))
        elif op == "rms_norm":
            w = np.ones((n,), np.float16)
            fn = ref_runner.prepare("rms_norm", x16, w, np.zeros_like(x16)) if use_tvm else (lambda: oracle.rms_norm(x16, w))
        else:
            fn = ref_runner.prepare("softmax", x16, np.zeros_like(x16)) if use_tvm else (lambda: oracle.softmax(x16))
        fn()
        return timed(fn, 3) * (m / rows), rows
    w = seeded_normal((n, k), 2, "float16", scale=0.02).numpy()
    if op == "gemv":
        x = seeded_normal((1, 1, k), 3, "float16").numpy()
        fn = ref_runner.prepare(f"gemv_n{n}_k{k}", x, w, np.zeros((1, 1, n), np.float16)) if use_tvm else (lambda: oracle.gemv(x, w))
        return timed(fn, 1), 1
    # gemm: rows so that the sample stays inside the budget (about 1 GFLOP/s/core for the TVM build)
    flop_row = 2.0 * n * k
    rate = 1.0e9 if use_tvm else 0.4e9 * max(1, oracle.max_threads())
    rows = int(max(1, min(m, budget_s * rate / flop_row)))
    x = seeded_normal((1, rows, k), 3, "float16").numpy()
    fn = ref_runner.prepare(f"gemm_n{n}_k{k}", x, w, np.zeros((1, rows, n), np.float16)) if use_tvm else (lambda: oracle.gemm_nt(x[0], w))
    return timed(fn, 1) * (m / rows), rows


def cpu_backend():
    """("reference", cores) when the TVM-built PrimFuncs can run here, else ("port", cores)."""
    import oracle
    try:
        from oracle import ref_runner
        ok, why = ref_runner.available()
    except Exception as e:  # noqa: BLE001
        ok, why = False, str(e)
    if ok:
        return "reference", 1, ""
    return "port", oracle.max_threads(), why


def cpu_sweep_seconds(budget_s):
    """Seconds one full step would take on the CPU, extrapolated from bounded samples."""
    backend, cores, why = cpu_backend()
    pts = sweep_points()
    per_gemm = budget_s / (2.0 * len([p for p in pts if p[0] == "gemm"]))
    total, sampled = 0.0, 0.0
    t_begin = time.perf_counter()
    for (op, m, n, k) in pts:
        s, _ = _cpu_point_time(op, m, n, k, backend, per_gemm)
        total += s
    sampled = time.perf_counter() - t_begin
    return total, backend, cores, why, sampled


def cpu_baseline(sample_seconds=15.0):
    from dtas_b200.profiling import measured_peaks
    peaks, _ = measured_peaks(ROOT)
    ideal_ns = sum(roofline_ns(*p, peaks)[0] for p in sweep_points())
    total_s, backend, cores, why, sampled = cpu_sweep_seconds(sample_seconds)
    return {"value": round(100.0 * ideal_ns * 1e-9 / total_s, 6), "unit": UNIT,
            "cores": cores, "kind": backend, "seconds_per_step_extrapolated": round(total_s, 1),
            "sample": (f"every point of the sweep on a bounded row slab (<=256 rows for elementwise/reductions, full GEMV, "
                       f"1-few rows per GEMM), scaled linearly to the full row count; {sampled:.1f} s of CPU work; "
                       + ("PrimFuncs built by TVM 0.23 (tilelang fork), target c, g++ -O3 -march=x86-64-v3, single thread"
                          if backend == "reference" else f"C port oracle/dtas_oracle.c with OpenMP ({why})"))}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    from dtas_b200.profiling import measured_peaks
    peaks, peak_src = measured_peaks(ROOT)
    ideal_ns = sum(roofline_ns(*p, peaks)[0] for p in sweep_points())
    budget = 8.0
    for _ in range(min(args.warmup, 1)):
        cpu_sweep_seconds(budget / 4)
    secs, backend, cores, why = [], "port", 1, ""
    for _ in range(max(1, min(args.steps, 3))):
        s, backend, cores, why, _ = cpu_sweep_seconds(budget)
        secs.append(s)
    s = sum(secs) / len(secs)
    value = round(100.0 * ideal_ns * 1e-9 / s, 6)
    unit = UNIT
    sample = ("each step: every point of the sweep timed on a bounded row slab and scaled linearly to its full row count; "
              + ("reference PrimFuncs built by TVM 0.23 (tilelang fork) for target c, g++ -O3 -march=x86-64-v3, single thread"
                 if backend == "reference" else f"C port oracle/dtas_oracle.c, OpenMP ({why})"))
    print(json.dumps({
        "impl": "reference", "metric": METRIC,
        "value": value, "unit": unit, "n_gpus": world, "steps": len(secs), "warmup": min(args.warmup, 1),
        "ms_per_step": round(s * 1e3, 1), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 (fp32 accumulate)", "data": "synthetic (seeded normal)",
        "config": bench_config(peaks, peak_src),
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": backend, "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="dtas_b200", choices=["dtas_b200", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the per-point graph-replay timings")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
