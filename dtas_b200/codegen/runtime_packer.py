"""Runtime module: what `Engine.tune_module` returns and `load_module_from_file` reloads.

The reference packs generated host code and a cubin into a `tvm.runtime.Module`
(python/dtas/codegen/runtime_packer.py:237-258) and reloads it from `work_dir`
(:260-283); users then call `rt_mod["cast"](x, y)` and
`rt_mod.time_evaluator("cast", dev, number=5, min_repeat_ms=50)`
(experiment/dtas_tuned/elementwise/cast/profile_cast.py:8-20).  Here the kernels already live
in libdtas_b200.so, so the module is the record of bound functions (operator, dtypes, static
dims, merged ranges, index table) stored as JSON in `work_dir`; reloading rebuilds nothing.
"""
import json
import os

from .. import _abi, ops
from ..profiling import time_op
from ..reference import torch_dtype
from ..workloads.spec import OpSpec

MODULE_FILE = "dtas_b200_module.json"


class BenchmarkResult:
    """Shape of TVM's time_evaluator result: `.mean`, `.min`, `.results` in seconds."""

    def __init__(self, t):
        self.mean = t["mean_us"] * 1e-6
        self.min = t["min_us"] * 1e-6
        self.results = [self.mean]
        self.launches = t["launches"]

    def __repr__(self):
        return f"BenchmarkResult(mean={self.mean * 1e6:.2f} us, min={self.min * 1e6:.2f} us, launches={self.launches})"


class PackedOp:
    """One bound function: destination-passing call on torch tensors."""

    def __init__(self, name, entry):
        self.name = name
        self.entry = entry
        self.spec = OpSpec.from_dict(entry["spec"])

    def bucket_index(self, m, m2=None):
        """Position in the range list that serves the symbolic dim(s): m, and m2 for a function with two
        (each clamped above its bound)."""
        table = self.entry["index_table"]
        if not table:
            return 0
        width = self.entry["range_div_factor"]
        if len(self.entry.get("dynamic_args", [])) == 2:
            starts = sorted({r["start"][1] for r in self.entry["ranges"]})
            n1 = len(starts)
            n0 = len(table) // n1
            i0 = min((m - 1) // width, n0 - 1)
            i1 = min(((m2 if m2 is not None else 1) - 1) // width, n1 - 1)
            return table[i0 * n1 + i1]
        return table[min((m - 1) // width, len(table) - 1)]

    def _expect(self, t, dtype, cols, what):
        if t.dtype != torch_dtype(dtype):
            raise _abi.DtasError(_abi.EINVAL, f"{self.name}: {what} must be {dtype}, got {t.dtype}")
        if cols and t.shape[-1] != cols:
            raise _abi.DtasError(_abi.EINVAL, f"{self.name}: {what} last dim must be {cols}, got {t.shape[-1]}")

    def __call__(self, *args):
        s = self.spec
        n_in = {"cast": 1, "copy": 1, "softmax": 1, "add": 2, "rms_norm": 2, "layer_norm": 3,
                "gemv": 2 + int(s.bias) + s.residuals, "gemm": 2 + int(s.bias) + s.residuals}[s.op]
        if len(args) != n_in + 1:
            raise _abi.DtasError(_abi.EINVAL, f"{self.name}: expected {n_in} input(s) and 1 output, got {len(args)} tensors")
        out = args[-1]
        if s.op in ("cast", "copy", "add", "rms_norm", "softmax", "layer_norm"):
            self._expect(args[0], s.in_dtype, s.cols, "input")
            self._expect(out, s.out_dtype, s.cols, "output")
        if s.op == "cast":
            return ops.cast(args[0], out)
        if s.op == "copy":
            return ops.copy(args[0], out)
        if s.op == "add":
            return ops.add(args[0], args[1], out)
        if s.op == "rms_norm":
            return ops.rms_norm(args[0], args[1], out, eps=s.eps)
        if s.op == "softmax":
            if s.cols == 0:      # symbolic reduction length: [..., m] -> rows x m
                if tuple(args[0].shape) != tuple(out.shape):
                    raise _abi.DtasError(_abi.EINVAL, f"{self.name}: input {tuple(args[0].shape)} and output {tuple(out.shape)} differ")
                cols = int(out.shape[-1])
                ops.softmax(args[0].reshape(-1, cols), out.view(-1, cols))
                return out
            return ops.softmax(args[0], out)
        if s.op == "layer_norm":
            return ops.layer_norm(args[0], args[1], args[2], out, eps=s.eps)
        if s.op in ("gemv", "gemm"):
            self._expect(args[0], "float16", s.k, "x")
            if tuple(args[1].shape) != (s.cols, s.k):
                raise _abi.DtasError(_abi.EINVAL, f"{self.name}: weight must be [{s.cols}, {s.k}], got {tuple(args[1].shape)}")
            # argument order of the reference's fused functions: x, W, bias, residuals..., out
            # (experiment/ModelIR/dolly-v2-3b-q0f16/before_dl.py:163)
            bias = args[2] if s.bias else None
            res = list(args[2 + int(s.bias):-1]) + [None, None]
            if out.dtype != torch_dtype(s.out_dtype):
                raise _abi.DtasError(_abi.EINVAL, f"{self.name}: output must be {s.out_dtype}, got {out.dtype}")
            fn = ops.gemv if s.op == "gemv" else ops.gemm_nt
            return fn(args[0], args[1], out, bias=bias, res1=res[0], res2=res[1], act=s.act or None)
        raise _abi.DtasError(_abi.EUNSUPPORTED, f"{self.name}: unknown op {s.op}")


class RuntimeModule:
    def __init__(self, record):
        _abi.lib()   # fail here, loudly, if the kernel library is missing
        self.record = record
        self._funcs = {name: PackedOp(name, e) for name, e in record["functions"].items()}
        # measured GEMM choices travel with the module: (re-)install them in the library
        for e in record["functions"].values():
            for row in e.get("measured_table", []):
                _abi.check(_abi.lib().dtas_gemm_table_set(e["spec"]["cols"], e["spec"]["k"], row["m_lo"], row["m_hi"],
                                                          row["bn"], row["split"]))

    def __getitem__(self, name):
        return self._funcs[name]

    get_function = __getitem__

    def __contains__(self, name):
        return name in self._funcs

    def keys(self):
        return self._funcs.keys()

    def time_evaluator(self, func_name, dev=None, number=5, min_repeat_ms=50, repeat=1):
        """Returns f(*tensors) -> BenchmarkResult; same knobs as TVM's time_evaluator."""
        fn = self._funcs[func_name]

        def evaluator(*args):
            t = time_op(lambda i: fn(*args), warmup=3, number=max(number, repeat), min_repeat_ms=min_repeat_ms)
            return BenchmarkResult(t)

        return evaluator


def load_module_from_file(work_dir: str) -> RuntimeModule:
    """Reloads the module `Engine(work_dir=...).tune_module` stored in work_dir."""
    path = os.path.join(work_dir, MODULE_FILE)
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path} not found: run Engine(work_dir=...).tune_module first")
    with open(path) as f:
        return RuntimeModule(json.load(f))
