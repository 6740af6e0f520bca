"""Builds oracle/_ref/dtas_ref_primfuncs.so: the workload PrimFuncs at the measured sizes,
compiled by TVM for the host CPU.  TEST / BASELINE INFRASTRUCTURE, not product.

The reference measures PrimFuncs that TVM builds; its own package cannot be imported against
the TVM of this image (it needs `tvm._ffi`, a CUDA-enabled TVM and $TVM_HOME), and this TVM
has no LLVM backend, so the PrimFuncs are built with target "c" and g++ -O3 -march=x86-64-v3
(AVX2 + F16C + FMA available, no FMA contraction of the PrimFunc arithmetic is relied on for parity:
this build is only timed).  -march=native is not used: the library is built on one machine and
timed on another.  The result needs the same
TVM runtime to load (oracle/ref_runner.py).  Nothing is copied from the reference tree: the
PrimFunc text comes from dtas_b200/workloads/tir_defs.py.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "dtas_ref_primfuncs.so")

GEMV_SHAPES = [(4096, 4096), (11008, 4096), (4096, 11008), (32000, 4096)]
GEMM_SHAPES = [(12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008)]


def ref_functions():
    from dtas_b200.workloads import tir_defs as td
    funcs = {
        "cast": td.cast(4096, "float32", "float16"),
        "add": td.add(11008, "float16"),
        "copy": td.copy(11008, "float16"),
        "rms_norm": td.rms_norm(4096, 1e-6),
        "softmax": td.softmax(4096, "float16"),
    }
    for n, k in GEMV_SHAPES:
        funcs[f"gemv_n{n}_k{k}"] = td.gemv(n, k)
    for n, k in GEMM_SHAPES:
        funcs[f"gemm_n{n}_k{k}"] = td.gemm_nt(n, k)
    return funcs


def build_all(quiet=False, force=False):
    if os.path.exists(REF_SO) and not force:
        src = os.path.join(ROOT, "dtas_b200", "workloads", "tir_defs.py")
        if os.path.getmtime(REF_SO) >= max(os.path.getmtime(src), os.path.getmtime(__file__)):
            return REF_SO
    from dtas_b200.workloads import tir_defs as td
    tvm = td._tvm()
    mod = td.make_module(ref_functions())
    lib = tvm.build(mod, target="c") if hasattr(tvm, "build") else tvm.compile(mod, target="c")
    os.makedirs(REF_DIR, exist_ok=True)
    lib.export_library(REF_SO, options=["-O3", "-march=x86-64-v3", "-Dhalf=_Float16"])
    if not quiet:
        print(f"built {REF_SO} with TVM {tvm.__version__} (target c)")
    return REF_SO


if __name__ == "__main__":
    build_all(force=True)
