"""Generates tests/golden/*.npz: outputs of the workload PrimFuncs built by TVM.

Run in a container that has a TVM (here: the fork bundled with tilelang, 0.23.dev0):
    python tests/golden/make_golden.py                    # every case
    python tests/golden/make_golden.py gemm_fused gemv    # only the cases of these operators
Each PrimFunc from dtas_b200/workloads/tir_defs.py is built for target "c", compiled with
g++ -O2 -Dhalf=_Float16 (TVM's own export_library), run on seeded inputs from
dtas_b200.reference.seeded_normal, and the output is stored.  Inputs are not stored: the
case list (golden_cases.py) holds their shapes, seeds and a CRC of their bytes, and the
tests regenerate them.
"""
import json
import os
import sys
import tempfile
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from dtas_b200.workloads import tir_defs as td  # noqa: E402
from tests.golden.golden_cases import CASES, make_inputs  # noqa: E402


def build(funcs):
    tvm = td._tvm()
    mod = td.make_module(funcs)
    lib = tvm.build(mod, target="c") if hasattr(tvm, "build") else tvm.compile(mod, target="c")
    path = os.path.join(tempfile.mkdtemp(), "golden.so")
    lib.export_library(path, options=["-O2", "-Dhalf=_Float16"])
    return tvm, tvm.runtime.load_module(path)


def prim_func(case):
    op, p = case["op"], case
    if op == "cast":
        return td.cast(p["H"], p["src"], p["dst"])
    if op == "add":
        return td.add(p["H"], p["dtype"])
    if op == "copy":
        return td.copy(p["H"], p["dtype"])
    if op == "rms_norm":
        return td.rms_norm(p["H"], p["eps"])
    if op == "softmax":
        return td.softmax(p["H"], p["dtype"])
    if op == "layer_norm":
        return td.layer_norm(p["H"], p["dtype"], p["eps"])
    if op == "softmax_dyn":
        return td.softmax_dynamic(p["heads"], p["dtype"])
    if op == "gemm":
        return td.gemm_nt(p["N"], p["K"])
    if op == "gemv":
        return td.gemv(p["N"], p["K"])
    if op in ("gemm_fused", "gemv_fused"):
        return td.matmul_fused(p["N"], p["K"], dynamic=op == "gemm_fused", bias=p.get("bias", True), act=p.get("act", ""),
                               residuals=p.get("residuals", 0), out_dtype=p.get("out", "float16"))
    raise ValueError(op)


def main():
    only = set(sys.argv[1:])
    outputs, meta = {}, {}
    meta_path = os.path.join(HERE, "golden_meta.json")
    if only and os.path.exists(meta_path):
        with open(meta_path) as f:
            meta = json.load(f)
    for name, case in CASES.items():
        if only and case["op"] not in only:
            continue
        tvm, rt = build({"f": prim_func(case)})
        ins, out = make_inputs(case)
        to_nd = tvm.runtime.tensor if hasattr(tvm.runtime, "tensor") else tvm.nd.array
        args = [to_nd(a) for a in ins] + [to_nd(out)]
        rt["f"](*args)
        res = args[-1].numpy()
        outputs[name] = res.reshape(-1, res.shape[-1])
        meta[name] = {"input_crc32": [zlib.crc32(np.ascontiguousarray(a).tobytes()) for a in ins]}
        print(name, res.shape, res.dtype)
    by_op = {}
    for name, arr in outputs.items():
        by_op.setdefault(CASES[name]["op"], {})[name] = arr
    for op, arrs in by_op.items():
        np.savez_compressed(os.path.join(HERE, f"{op}.npz"), **arrs)
    tvm = td._tvm()
    meta["_generator"] = {"tvm": tvm.__version__, "target": "c", "cc_options": ["-O2", "-Dhalf=_Float16"]}
    with open(meta_path, "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)


if __name__ == "__main__":
    main()
