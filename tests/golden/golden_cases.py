"""Case list of the golden fixtures: operator, static sizes, row count, seeds.

Shared by make_golden.py (which produces the outputs with TVM) and the tests (which
regenerate the same inputs and compare).  Input k of a case is
seeded_normal(shape, seed + k, ...).
"""
import numpy as np

from dtas_b200.reference import seeded_normal

CASES = {
    # elementwise -----------------------------------------------------------------------
    "cast_f32_f16_m1": dict(op="cast", src="float32", dst="float16", H=4096, m=1, seed=0),
    "cast_f32_f16_m17": dict(op="cast", src="float32", dst="float16", H=4096, m=17, seed=0),
    "cast_f32_f16_odd": dict(op="cast", src="float32", dst="float16", H=101, m=5, seed=11),
    "cast_f16_f32_m3": dict(op="cast", src="float16", dst="float32", H=2560, m=3, seed=12),
    "add_f16_m1": dict(op="add", dtype="float16", H=11008, m=1, seed=1000),
    "add_f16_m7": dict(op="add", dtype="float16", H=11008, m=7, seed=1000),
    "add_f32_m2": dict(op="add", dtype="float32", H=2560, m=2, seed=1010),
    "add_i8_m3": dict(op="add", dtype="int8", H=2560, m=3, seed=1020),
    "copy_f16_m7": dict(op="copy", dtype="float16", H=11008, m=7, seed=1000),
    # row reductions --------------------------------------------------------------------
    "rms_norm_m1": dict(op="rms_norm", H=4096, m=1, eps=1e-6, seed=2000),
    "rms_norm_m33": dict(op="rms_norm", H=4096, m=33, eps=1e-6, seed=2000),
    "softmax_m1": dict(op="softmax", dtype="float16", H=4096, m=1, seed=2000),
    "softmax_m33": dict(op="softmax", dtype="float16", H=4096, m=33, seed=2000),
    "softmax_f32_m4": dict(op="softmax", dtype="float32", H=1000, m=4, seed=2030),
    "layer_norm_f32_m3": dict(op="layer_norm", dtype="float32", H=2560, m=3, eps=1e-5, seed=2040),
    "softmax_dyn_f32_h32_n5_m77": dict(op="softmax_dyn", dtype="float32", heads=32, n=5, m=77, seed=2050),
    "softmax_dyn_f32_h32_n3_m256": dict(op="softmax_dyn", dtype="float32", heads=32, n=3, m=256, seed=2060),
    # gemv: the four Llama-2-7B shapes ------------------------------------------------------
    "gemv_4096_4096": dict(op="gemv", N=4096, K=4096, seed=3000),
    "gemv_11008_4096": dict(op="gemv", N=11008, K=4096, seed=3010),
    "gemv_4096_11008": dict(op="gemv", N=4096, K=11008, seed=3020),
    "gemv_32000_4096": dict(op="gemv", N=32000, K=4096, seed=3030),
    # gemm --------------------------------------------------------------------------------
    "gemm_m16_4096_4096": dict(op="gemm", m=16, N=4096, K=4096, seed=4000),
    "gemm_m255_384_1024": dict(op="gemm", m=255, N=384, K=1024, seed=4010),
    "gemm_m64_200_264": dict(op="gemm", m=64, N=200, K=264, seed=4020),
    # fused matmul tails of the model workloads (bias / gelu / two residuals / trailing cast) ---------
    "gemm_bias_m33_384_512": dict(op="gemm_fused", m=33, N=384, K=512, seed=5000),
    "gemm_gelu_m33_384_512": dict(op="gemm_fused", m=33, N=384, K=512, act="gelu", seed=5010),
    "gemm_res2_m65_200_264": dict(op="gemm_fused", m=65, N=200, K=264, residuals=2, seed=5020),
    "gemm_res2_cast_m16_512_1024": dict(op="gemm_fused", m=16, N=512, K=1024, residuals=2, out="float32", seed=5030),
    "gemm_res1_nobias_m300_256_128": dict(op="gemm_fused", m=300, N=256, K=128, bias=False, residuals=1, seed=5040),
    "gemv_bias_2560_10240": dict(op="gemv_fused", N=2560, K=10240, seed=6000),
    "gemv_gelu_10240_2560": dict(op="gemv_fused", N=10240, K=2560, act="gelu", seed=6010),
    "gemv_res2_2560_2560": dict(op="gemv_fused", N=2560, K=2560, residuals=2, seed=6020),
    "gemv_res2_cast_2560_2560": dict(op="gemv_fused", N=2560, K=2560, residuals=2, out="float32", seed=6030),
}


def make_inputs(case):
    """-> ([numpy inputs], numpy output buffer) in the PrimFunc's argument order."""
    op, s = case["op"], case["seed"]

    def nd(shape, k, dtype, **kw):
        return seeded_normal(shape, s + k, dtype, **kw).numpy()

    if op == "cast":
        m, h = case["m"], case["H"]
        return [nd((1, m, h), 0, case["src"])], np.zeros((1, m, h), case["dst"])
    if op == "add":
        m, h, dt = case["m"], case["H"], case["dtype"]
        return [nd((1, m, h), 0, dt), nd((1, m, h), 1, dt)], np.zeros((1, m, h), dt)
    if op == "copy":
        m, h, dt = case["m"], case["H"], case["dtype"]
        return [nd((1, m, h), 0, dt)], np.zeros((1, m, h), dt)
    if op == "rms_norm":
        m, h = case["m"], case["H"]
        return [nd((1, m, h), 0, "float16"), nd((h,), 1, "float16", scale=0.1, mean=1.0)], np.zeros((1, m, h), "float16")
    if op == "softmax":
        m, h = case["m"], case["H"]
        return [nd((1, m, h), 0, case["dtype"])], np.zeros((1, m, h), "float16")
    if op == "softmax_dyn":
        shape = (1, case["heads"], case["n"], case["m"])
        return [nd(shape, 0, case["dtype"], scale=3.0)], np.zeros(shape, "float16")
    if op == "layer_norm":
        m, h = case["m"], case["H"]
        return [nd((1, m, h), 0, case["dtype"]), nd((h,), 1, "float32", scale=0.1, mean=1.0),
                nd((h,), 2, "float32", scale=0.1)], np.zeros((1, m, h), "float16")
    if op == "gemv":
        n, k = case["N"], case["K"]
        return [nd((1, 1, k), 0, "float16"), nd((n, k), 1, "float16", scale=0.02)], np.zeros((1, 1, n), "float16")
    if op == "gemm":
        m, n, k = case["m"], case["N"], case["K"]
        return [nd((1, m, k), 0, "float16"), nd((n, k), 1, "float16", scale=0.02)], np.zeros((1, m, n), "float16")
    if op in ("gemm_fused", "gemv_fused"):
        m = case["m"] if op == "gemm_fused" else 1
        n, k = case["N"], case["K"]
        ins = [nd((1, m, k), 0, "float16"), nd((n, k), 1, "float16", scale=0.02)]
        if case.get("bias", True):
            ins.append(nd((n,), 2, "float16", scale=0.5))
        for r in range(case.get("residuals", 0)):
            ins.append(nd((1, m, n), 3 + r, "float16"))
        return ins, np.zeros((1, m, n), case.get("out", "float16"))
    raise ValueError(op)
