"""TVMScript builders for the workload PrimFuncs.

Same style as the reference's workload files: one PrimFunc per operator, the symbolic dim
declared as `n = T.int64()`, buffers shaped `(1, n, H)`, "tir.noalias" set
(tuning_test/tune_cast.py:10-21, tune_ele_add.py:10-22, tune_ele_copy.py:10-21;
experiment/dtas_tuned/general_reduction/{layernorm,softmax}/profile_dlight.py;
experiment/testIR/GEMM/dlight.py:30-50; experiment/testIR/GEMV/m1n2560k10240/dlight_gemv.py:8-27).
The static sizes and dtypes are parameters, because the measured configurations use
Llama-2-7B sizes where the reference used dolly-v2-3b's 2560.

Differences from the reference text, all dictated by the configurations being measured:
  * reductions read fp16 (`T.Cast("float32", x)` on every load) as well as fp32;
  * `rms_norm` does not exist in the reference; it reuses the layer-norm block structure
    (one "SSR" reduction block, one injective epilogue block);
  * matmul blocks accumulate in fp32 and cast once (the reference accumulates in fp16).

Requires an importable `tvm` (for example the one bundled with tilelang:
`import tilelang; from tilelang import tvm`).  Nothing else in dtas_b200 needs TVM.
"""


def _tvm():
    try:
        import tvm  # noqa: F401
    except ImportError:
        import tilelang  # noqa: F401
        from tilelang import tvm  # noqa: F401
    import tvm
    return tvm


def cast(H, src="float32", dst="float16", name="cast"):
    _tvm()
    from tvm.script import tir as T

    @T.prim_func
    def func(var_A: T.handle, var_compute: T.handle):
        T.func_attr({"global_symbol": name, "tir.noalias": True})
        n = T.int64()
        A = T.match_buffer(var_A, (T.int64(1), n, T.int64(H)), src)
        compute = T.match_buffer(var_compute, (T.int64(1), n, T.int64(H)), dst)
        for i0, i1, i2 in T.grid(T.int64(1), n, T.int64(H)):
            with T.block("compute"):
                v_i0, v_i1, v_i2 = T.axis.remap("SSS", [i0, i1, i2])
                T.reads(A[v_i0, v_i1, v_i2])
                T.writes(compute[v_i0, v_i1, v_i2])
                compute[v_i0, v_i1, v_i2] = T.Cast(dst, A[v_i0, v_i1, v_i2])

    return func


def add(H, dtype="float16", name="add"):
    _tvm()
    from tvm.script import tir as T

    @T.prim_func
    def func(var_A: T.handle, var_B: T.handle, var_T_add: T.handle):
        T.func_attr({"global_symbol": name, "op_pattern": 0, "tir.noalias": True})
        n = T.int64()
        A = T.match_buffer(var_A, (T.int64(1), n, T.int64(H)), dtype)
        B = T.match_buffer(var_B, (T.int64(1), n, T.int64(H)), dtype)
        T_add = T.match_buffer(var_T_add, (T.int64(1), n, T.int64(H)), dtype)
        for ax0, ax1, ax2 in T.grid(T.int64(1), n, T.int64(H)):
            with T.block("T_add"):
                v_ax0, v_ax1, v_ax2 = T.axis.remap("SSS", [ax0, ax1, ax2])
                T.reads(A[v_ax0, v_ax1, v_ax2], B[v_ax0, v_ax1, v_ax2])
                T.writes(T_add[v_ax0, v_ax1, v_ax2])
                T_add[v_ax0, v_ax1, v_ax2] = A[v_ax0, v_ax1, v_ax2] + B[v_ax0, v_ax1, v_ax2]

    return func


def copy(H, dtype="float16", name="copy"):
    _tvm()
    from tvm.script import tir as T

    @T.prim_func
    def func(var_A: T.handle, var_B: T.handle):
        T.func_attr({"global_symbol": name, "op_pattern": 0, "tir.noalias": True})
        n = T.int64()
        A = T.match_buffer(var_A, (T.int64(1), n, T.int64(H)), dtype)
        B = T.match_buffer(var_B, (T.int64(1), n, T.int64(H)), dtype)
        for ax0, ax1, ax2 in T.grid(T.int64(1), n, T.int64(H)):
            with T.block("T_copy"):
                v_ax0, v_ax1, v_ax2 = T.axis.remap("SSS", [ax0, ax1, ax2])
                T.reads(A[v_ax0, v_ax1, v_ax2])
                T.writes(B[v_ax0, v_ax1, v_ax2])
                B[v_ax0, v_ax1, v_ax2] = A[v_ax0, v_ax1, v_ax2]

    return func


def rms_norm(H, eps=1e-6, name="rms_norm"):
    _tvm()
    from tvm.script import tir as T
    inv_h = 1.0 / H

    @T.prim_func
    def func(var_x: T.handle, weight: T.Buffer((T.int64(H),), "float16"), var_y: T.handle):
        T.func_attr({"global_symbol": name, "tir.noalias": True})
        n = T.int64()
        x = T.match_buffer(var_x, (T.int64(1), n, T.int64(H)), "float16")
        y = T.match_buffer(var_y, (T.int64(1), n, T.int64(H)), "float16")
        sq_sum = T.alloc_buffer((T.int64(1), n))
        for ax0, ax1, k2 in T.grid(T.int64(1), n, T.int64(H)):
            with T.block("sq_sum"):
                v_ax0, v_ax1, v_k2 = T.axis.remap("SSR", [ax0, ax1, k2])
                T.reads(x[v_ax0, v_ax1, v_k2])
                T.writes(sq_sum[v_ax0, v_ax1])
                with T.init():
                    sq_sum[v_ax0, v_ax1] = T.float32(0)
                sq_sum[v_ax0, v_ax1] = sq_sum[v_ax0, v_ax1] + T.Cast("float32", x[v_ax0, v_ax1, v_k2]) * T.Cast("float32", x[v_ax0, v_ax1, v_k2])
        for ax0, ax1, ax2 in T.grid(T.int64(1), n, T.int64(H)):
            with T.block("T_rms_norm"):
                v_ax0, v_ax1, v_ax2 = T.axis.remap("SSS", [ax0, ax1, ax2])
                T.reads(x[v_ax0, v_ax1, v_ax2], sq_sum[v_ax0, v_ax1], weight[v_ax2])
                T.writes(y[v_ax0, v_ax1, v_ax2])
                y[v_ax0, v_ax1, v_ax2] = T.Cast("float16", T.Cast("float32", x[v_ax0, v_ax1, v_ax2]) * T.rsqrt(sq_sum[v_ax0, v_ax1] * T.float32(inv_h) + T.float32(eps)) * T.Cast("float32", weight[v_ax2]))

    return func


def softmax(H, in_dtype="float16", name="softmax"):
    """fused_softmax_cast with the row count symbolic and the reduced length H static."""
    _tvm()
    from tvm.script import tir as T

    @T.prim_func
    def func(p_A: T.handle, p_output0: T.handle):
        T.func_attr({"global_symbol": name, "tir.noalias": True})
        n = T.int64()
        A = T.match_buffer(p_A, (T.int64(1), n, T.int64(H)), in_dtype)
        compute_intermediate = T.match_buffer(p_output0, (T.int64(1), n, T.int64(H)), "float16")
        T_softmax_maxelem = T.alloc_buffer((T.int64(1), n))
        T_softmax_exp = T.alloc_buffer((T.int64(1), n, T.int64(H)))
        T_softmax_expsum = T.alloc_buffer((T.int64(1), n))
        for i0, i1, k in T.grid(T.int64(1), n, T.int64(H)):
            with T.block("T_softmax_maxelem"):
                v_i0, v_i1, v_k = T.axis.remap("SSR", [i0, i1, k])
                with T.init():
                    T_softmax_maxelem[v_i0, v_i1] = T.float32(-3.4028234663852886e+38)
                T_softmax_maxelem[v_i0, v_i1] = T.max(T_softmax_maxelem[v_i0, v_i1], T.Cast("float32", A[v_i0, v_i1, v_k]))
        for i0, i1, i2 in T.grid(T.int64(1), n, T.int64(H)):
            with T.block("T_softmax_exp"):
                v_i0, v_i1, v_i2 = T.axis.remap("SSS", [i0, i1, i2])
                T_softmax_exp[v_i0, v_i1, v_i2] = T.exp(T.Cast("float32", A[v_i0, v_i1, v_i2]) - T_softmax_maxelem[v_i0, v_i1])
        for i0, i1, k in T.grid(T.int64(1), n, T.int64(H)):
            with T.block("T_softmax_expsum"):
                v_i0, v_i1, v_k = T.axis.remap("SSR", [i0, i1, k])
                with T.init():
                    T_softmax_expsum[v_i0, v_i1] = T.float32(0)
                T_softmax_expsum[v_i0, v_i1] = T_softmax_expsum[v_i0, v_i1] + T_softmax_exp[v_i0, v_i1, v_k]
        for i0, i1, i2 in T.grid(T.int64(1), n, T.int64(H)):
            with T.block("compute"):
                v_i0, v_i1, v_i2 = T.axis.remap("SSS", [i0, i1, i2])
                compute_intermediate[v_i0, v_i1, v_i2] = T.Cast("float16", T_softmax_exp[v_i0, v_i1, v_i2] / T_softmax_expsum[v_i0, v_i1])

    return func


def layer_norm(H, in_dtype="float32", eps=1e-5, name="layer_norm"):
    """fused_layer_norm_cast: sum and sum of squares in one reduction block, fp32 gamma/beta."""
    _tvm()
    from tvm.script import tir as T
    inv_h = 1.0 / H

    @T.prim_func
    def func(p_x: T.handle, gamma: T.Buffer((T.int64(H),), "float32"), beta: T.Buffer((T.int64(H),), "float32"), p_output0: T.handle):
        T.func_attr({"global_symbol": name, "tir.noalias": True})
        n = T.int64()
        x = T.match_buffer(p_x, (T.int64(1), n, T.int64(H)), in_dtype)
        out = T.match_buffer(p_output0, (T.int64(1), n, T.int64(H)), "float16")
        red_v0 = T.alloc_buffer((T.int64(1), n))
        red_v1 = T.alloc_buffer((T.int64(1), n))
        for ax0, ax1, k2 in T.grid(T.int64(1), n, T.int64(H)):
            with T.block("A_red_temp"):
                v_ax0, v_ax1, v_k2 = T.axis.remap("SSR", [ax0, ax1, k2])
                with T.init():
                    red_v0[v_ax0, v_ax1] = T.float32(0)
                    red_v1[v_ax0, v_ax1] = T.float32(0)
                v0: T.float32 = red_v0[v_ax0, v_ax1] + T.Cast("float32", x[v_ax0, v_ax1, v_k2])
                v1: T.float32 = red_v1[v_ax0, v_ax1] + T.Cast("float32", x[v_ax0, v_ax1, v_k2]) * T.Cast("float32", x[v_ax0, v_ax1, v_k2])
                red_v0[v_ax0, v_ax1] = v0
                red_v1[v_ax0, v_ax1] = v1
        for ax0, ax1, ax2 in T.grid(T.int64(1), n, T.int64(H)):
            with T.block("T_layer_norm"):
                v_ax0, v_ax1, v_ax2 = T.axis.remap("SSS", [ax0, ax1, ax2])
                out[v_ax0, v_ax1, v_ax2] = T.Cast("float16", (T.Cast("float32", x[v_ax0, v_ax1, v_ax2]) - red_v0[v_ax0, v_ax1] * T.float32(inv_h)) * T.rsqrt(red_v1[v_ax0, v_ax1] * T.float32(inv_h) - red_v0[v_ax0, v_ax1] * T.float32(inv_h) * (red_v0[v_ax0, v_ax1] * T.float32(inv_h)) + T.float32(eps)) * gamma[v_ax2] + beta[v_ax2])

    return func


def gemm_nt(N, K, name="NT_matmul"):
    """Y[1, n, N] = X[1, n, K] . W[N, K]^T, fp16 operands, fp32 accumulator, fp16 result."""
    _tvm()
    from tvm.script import tir as T

    @T.prim_func
    def func(p_x: T.handle, w: T.Buffer((T.int64(N), T.int64(K)), "float16"), p_output0: T.handle):
        T.func_attr({"global_symbol": name, "tir.noalias": True})
        n = T.int64()
        x = T.match_buffer(p_x, (T.int64(1), n, T.int64(K)), "float16")
        y = T.match_buffer(p_output0, (T.int64(1), n, T.int64(N)), "float16")
        acc = T.alloc_buffer((T.int64(1), n, T.int64(N)), "float32")
        for i0, i1, i2, k in T.grid(T.int64(1), n, T.int64(N), T.int64(K)):
            with T.block("NT_matmul"):
                v_i0, v_i1, v_i2, v_k = T.axis.remap("SSSR", [i0, i1, i2, k])
                T.reads(x[v_i0, v_i1, v_k], w[v_i2, v_k])
                T.writes(acc[v_i0, v_i1, v_i2])
                with T.init():
                    acc[v_i0, v_i1, v_i2] = T.float32(0)
                acc[v_i0, v_i1, v_i2] = acc[v_i0, v_i1, v_i2] + T.Cast("float32", x[v_i0, v_i1, v_k]) * T.Cast("float32", w[v_i2, v_k])
        for ax0, ax1, ax2 in T.grid(T.int64(1), n, T.int64(N)):
            with T.block("compute"):
                v_ax0, v_ax1, v_ax2 = T.axis.remap("SSS", [ax0, ax1, ax2])
                y[v_ax0, v_ax1, v_ax2] = T.Cast("float16", acc[v_ax0, v_ax1, v_ax2])

    return func


def gemv(N, K, name="gemv"):
    """y[1, 1, N] = x[1, 1, K] . W[N, K]^T, no symbolic dim (decode step), fp32 accumulator."""
    _tvm()
    from tvm.script import tir as T

    @T.prim_func
    def func(x: T.Buffer((1, 1, K), "float16"), w: T.Buffer((N, K), "float16"), y: T.Buffer((1, 1, N), "float16")):
        T.func_attr({"global_symbol": name, "tir.noalias": True})
        acc = T.alloc_buffer((1, 1, N), "float32")
        for i0, i1, i2, k in T.grid(1, 1, N, K):
            with T.block("NT_matmul"):
                v_i0, v_i1, v_i2, v_k = T.axis.remap("SSSR", [i0, i1, i2, k])
                T.reads(x[v_i0, v_i1, v_k], w[v_i2, v_k])
                T.writes(acc[v_i0, v_i1, v_i2])
                with T.init():
                    acc[v_i0, v_i1, v_i2] = T.float32(0)
                acc[v_i0, v_i1, v_i2] = acc[v_i0, v_i1, v_i2] + T.Cast("float32", x[v_i0, v_i1, v_k]) * T.Cast("float32", w[v_i2, v_k])
        for ax0, ax1, ax2 in T.grid(1, 1, N):
            with T.block("compute"):
                v_ax0, v_ax1, v_ax2 = T.axis.remap("SSS", [ax0, ax1, ax2])
                y[v_ax0, v_ax1, v_ax2] = T.Cast("float16", acc[v_ax0, v_ax1, v_ax2])

    return func


def softmax_dynamic(heads=32, dtype="float32", name="fused_softmax_cast"):
    """Softmax over a symbolic last dim, cast to fp16: the attention-score form
    fused_softmax_cast3 of experiment/ModelIR/dolly-v2-3b-q0f16/before_dl.py:756-800
    (x [1, heads, n, m] -> max over m, exp(x - max), sum, divide, cast), two symbolic dims."""
    _tvm()
    from tvm import te, tir
    n, m = te.var("n", "int64"), te.var("m", "int64")
    shape = (1, heads, n, m)
    x = te.placeholder(shape, dtype, name="lv_scores")
    k1 = te.reduce_axis((0, m), name="k")
    mx = te.compute((1, heads, n), lambda i0, i1, i2: te.max(x[i0, i1, i2, k1].astype("float32"), axis=k1), name="T_softmax_maxelem")
    ex = te.compute(shape, lambda i0, i1, i2, i3: tir.exp(x[i0, i1, i2, i3].astype("float32") - mx[i0, i1, i2]), name="T_softmax_exp")
    k2 = te.reduce_axis((0, m), name="k")
    sm = te.compute((1, heads, n), lambda i0, i1, i2: te.sum(ex[i0, i1, i2, k2], axis=k2), name="T_softmax_expsum")
    nr = te.compute(shape, lambda i0, i1, i2, i3: ex[i0, i1, i2, i3] / sm[i0, i1, i2], name="T_softmax_norm")
    out = te.compute(shape, lambda i0, i1, i2, i3: nr[i0, i1, i2, i3].astype("float16"), name="compute")
    return te.create_prim_func([x, out]).with_attr("global_symbol", name)


def matmul_fused(N, K, dynamic=True, bias=True, act="", residuals=0, out_dtype="float16", name="fused_NT_matmul"):
    """The fused matmul forms of the reference's model workloads
    (experiment/ModelIR/dolly-v2-3b-q0f16/before_dl.py: fused_NT_matmul_add :552,
    fused_NT_matmul3_add2_gelu :248, fused_NT_matmul2_add1_add3_add3 :163, ..._cast :202, and the
    decode-time forms with a static single row :96, :408, :442, :483), block by block:
    matmul -> + bias -> [* 1/sqrt(2) -> erf in fp32 -> * 0.5 -> 0.5 + -> *] -> res1 + -> + res2 -> [cast].
    Every block after the matmul stores fp16, as in the reference; the matmul itself accumulates
    in fp32 and is rounded to fp16 once (the reference accumulates in fp16).  Arguments:
    x, W, [bias], [res1], [res2], out.  Built with te.create_prim_func so that the optional
    stages are plain Python conditions."""
    tvm = _tvm()
    from tvm import te, tir
    rows = te.var("n", "int64") if dynamic else 1
    shape = (1, rows, N)
    x = te.placeholder((1, rows, K), "float16", name="lv_x")
    w = te.placeholder((N, K), "float16", name="param_w")
    args = [x, w]
    k = te.reduce_axis((0, K), name="k")
    acc = te.compute(shape, lambda i0, i1, i2: te.sum(x[i0, i1, k].astype("float32") * w[i2, k].astype("float32"), axis=k),
                     name="NT_matmul")
    t = te.compute(shape, lambda i0, i1, i2: acc[i0, i1, i2].astype("float16"), name="NT_matmul_intermediate")
    if bias:
        b = te.placeholder((N,), "float16", name="param_bias")
        args.append(b)
        prev = t
        t = te.compute(shape, lambda i0, i1, i2: prev[i0, i1, i2] + b[i2], name="T_add")
    if act == "gelu":
        base = t
        u = te.compute(shape, lambda i0, i1, i2: base[i0, i1, i2] * tir.const(0.70710678118654757, "float16"), name="T_multiply")
        c0 = te.compute(shape, lambda i0, i1, i2: u[i0, i1, i2].astype("float32"), name="compute")
        c1 = te.compute(shape, lambda i0, i1, i2: tir.erf(c0[i0, i1, i2]), name="compute_1")
        c2 = te.compute(shape, lambda i0, i1, i2: c1[i0, i1, i2].astype("float16"), name="compute_2")
        m1 = te.compute(shape, lambda i0, i1, i2: c2[i0, i1, i2] * tir.const(0.5, "float16"), name="T_multiply_1")
        a1 = te.compute(shape, lambda i0, i1, i2: tir.const(0.5, "float16") + m1[i0, i1, i2], name="T_add_gelu")
        t = te.compute(shape, lambda i0, i1, i2: base[i0, i1, i2] * a1[i0, i1, i2], name="T_multiply_2")
    elif act:
        raise ValueError(f"unknown activation {act!r}")
    def add_stage(lhs, rhs, stage):
        return te.compute(shape, lambda i0, i1, i2: lhs[i0, i1, i2] + rhs[i0, i1, i2], name=stage)

    for r in range(residuals):
        res = te.placeholder(shape, "float16", name=f"lv_res{r + 1}")
        args.append(res)
        # the reference adds the first residual on the left, the second on the right
        t = add_stage(res, t, "T_add_1") if r == 0 else add_stage(t, res, "T_add_2")
    if out_dtype != "float16":
        prev = t
        t = te.compute(shape, lambda i0, i1, i2: prev[i0, i1, i2].astype(out_dtype), name="compute_cast")
    args.append(t)
    func = te.create_prim_func(args)
    return func.with_attr("global_symbol", name)


def make_module(funcs, upper_bound=None):
    """IRModule from {name: PrimFunc}; `upper_bound` mirrors the reference's
    `tir_var_upper_bound` function attribute (tuning_test/tune_cast.py:27)."""
    tvm = _tvm()
    out = {}
    for name, f in funcs.items():
        if upper_bound is not None:
            f = f.with_attr("tir_var_upper_bound", {"n": upper_bound})
        out[name] = f.with_attr("global_symbol", name)
    return tvm.IRModule(out)
