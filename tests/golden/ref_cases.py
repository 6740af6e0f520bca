"""Case list of the fixtures made from the reference's own PrimFunc text.

Each entry names the reference file that holds an `@I.ir_module class Module`, the PrimFunc in it,
and the seeded inputs it is run on.  `make_ref_golden.py` parses that text with TVM, builds it for
the CPU and stores the outputs; the tests regenerate the same inputs from the seeds below.

Shapes are the reference's own (hidden size 2560, `[1, n, 2560]` buffers, 1000 rows of symbolic
length for the softmax); `n` takes values on both sides of the 256-wide bucket boundary.  Inputs
are the seeded normal tensors of the measured configurations rather than the reference's
uniform(0, 1) draws: with fp16 accumulation (which the reference's matmul PrimFuncs use) a sum
of 2560 uniform products near 640 has an fp16 spacing of 0.5 and pins nothing.
"""
import numpy as np

from dtas_b200.reference import seeded_normal

H = 2560
N_VALUES = (1, 17, 256, 257, 1025)

# key -> reference file (relative to the reference tree), PrimFunc name, operator class
SOURCES = {
    "cast": dict(path="tuning_test/tune_cast.py", func="cast", op="cast"),
    "add": dict(path="tuning_test/tune_ele_add.py", func="add", op="add"),
    "copy": dict(path="tuning_test/tune_ele_copy.py", func="copy", op="copy"),
    "layer_norm": dict(path="experiment/dtas_tuned/general_reduction/layernorm/profile_dlight.py",
                       func="fused_layer_norm_cast", op="layer_norm"),
    "softmax": dict(path="experiment/dtas_tuned/general_reduction/softmax/profile_dlight.py",
                    func="fused_softmax_cast", op="softmax"),
    "gemm": dict(path="experiment/testIR/GEMM/dlight.py", func="main", op="gemm"),
    "gemv": dict(path="experiment/testIR/GEMV/m1n2560k10240/dlight_gemv.py", func="main", op="gemv"),
}

SEED0 = {"cast": 7000, "add": 7100, "copy": 7200, "layer_norm": 7300, "softmax": 7400, "gemm": 7500, "gemv": 7600}

# operators whose outputs are compared bit for bit: the whole output is pinned by a SHA-256
EXACT = ("cast", "add", "copy")


def n_values(key):
    return (1,) if key == "gemv" else N_VALUES      # the GEMV PrimFunc has no symbolic dim


def make_inputs(key, n):
    """-> ([numpy inputs], zeroed numpy output) in the PrimFunc's argument order."""
    s = SEED0[key] + 10 * N_VALUES.index(n) if n in N_VALUES else SEED0[key]

    def nd(shape, k, dtype, **kw):
        return seeded_normal(shape, s + k, dtype, **kw).numpy()

    if key == "cast":       # fp16 -> fp32
        return [nd((1, n, H), 0, "float16")], np.zeros((1, n, H), "float32")
    if key == "add":        # int8, wraps around
        return [nd((1, n, H), 0, "int8"), nd((1, n, H), 1, "int8")], np.zeros((1, n, H), "int8")
    if key == "copy":       # fp32
        return [nd((1, n, H), 0, "float32")], np.zeros((1, n, H), "float32")
    if key == "layer_norm":  # fp32 in, fp32 gamma / beta, fp16 out
        return [nd((1, n, H), 0, "float32"), nd((H,), 1, "float32", scale=0.1, mean=1.0),
                nd((H,), 2, "float32", scale=0.1)], np.zeros((1, n, H), "float16")
    if key == "softmax":    # 1000 rows of symbolic length n, fp32 in, fp16 out
        return [nd((1, 1000, n), 0, "float32", scale=3.0)], np.zeros((1, 1000, n), "float16")
    if key == "gemm":       # [1, n, 2560] x [10240, 2560]^T + bias, fp16 accumulation
        return [nd((1, n, H), 0, "float16"), seeded_normal((10240, H), SEED0[key] + 1, "float16", scale=0.02).numpy(),
                seeded_normal((10240,), SEED0[key] + 2, "float16", scale=0.5).numpy()], np.zeros((1, n, 10240), "float16")
    if key == "gemv":       # [1, 1, 10240] x [2560, 10240]^T + bias, fp16 accumulation
        return [nd((1, 1, 10240), 0, "float16"), nd((H, 10240), 1, "float16", scale=0.02),
                nd((H,), 2, "float16", scale=0.5)], np.zeros((1, 1, H), "float16")
    raise KeyError(key)


def stored_rows(key, n_rows):
    """Row indices of the [rows, cols] output that the fixture keeps (all rows when there are few):
    first, last and both sides of every multiple of 256, so the tails of every kernel layout are seen."""
    limit = 32 if key in EXACT or key in ("layer_norm", "softmax") else 12
    if n_rows <= limit:
        return list(range(n_rows))
    picks = {0, 1, n_rows - 2, n_rows - 1, n_rows // 2, n_rows // 3}
    for b in range(256, n_rows, 256):
        picks.update((b - 1, b))
    return sorted(p for p in picks if 0 <= p < n_rows)[:limit]
