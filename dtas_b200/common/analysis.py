"""Classification of a workload function into an operator class and a kernel binding.

The reference classifies a PrimFunc as GEMM / GEMV / Reduction / Elementwise after
normalising its blocks with a TIR schedule (python/dtas/common/analisys.py:333-458; kinds at
:49-55; at most two dynamic dims, :353-366).  Only that contract is kept here: given a
PrimFunc (when a TVM is importable) or an OpSpec, produce the FuncKind, the dynamic
arguments, whether fp16 is used, and the OpSpec the runtime binds to a kernel.  The analysis
walks the PrimFunc's blocks directly - iterator kinds, the expression stored by each block,
buffer shapes and dtypes - instead of rewriting it with schedule primitives.
"""
from enum import Enum

from ..workloads.spec import OpSpec


class FuncKind(Enum):
    kFunc_GEMM = 0
    kFunc_GEMV = 1
    kFunc_Reduction = 2
    kFunc_Elementwise = 3
    kFunc_Transpose = 4
    KFunc_Fallback = 5


_KIND_OF = {"gemm": FuncKind.kFunc_GEMM, "gemv": FuncKind.kFunc_GEMV,
            "reduction": FuncKind.kFunc_Reduction, "elementwise": FuncKind.kFunc_Elementwise}


class UnsupportedWorkload(ValueError):
    """The function does not map onto one of the operator classes of this library."""


def _static(dim):
    """int value of a static dim, None for a symbolic one."""
    try:
        return int(dim)
    except TypeError:
        return None


class _BlockFacts:
    def __init__(self, block):
        self.name = block.name_hint
        self.iter_types = [int(iv.iter_type) for iv in block.iter_vars]
        self.has_reduce = any(t == 2 for t in self.iter_types)   # IterVar.CommReduce
        self.block = block


def _collect_blocks(func):
    from tvm import tir
    from tvm.tir import stmt_functor
    blocks = []

    def visit(node):
        if isinstance(node, tir.Block) and node.name_hint != "root" and len(node.iter_vars) > 0:
            blocks.append(_BlockFacts(node))

    stmt_functor.post_order_visit(func.body, visit)
    return blocks


def _calls_and_ops(stmt):
    """Names of intrinsic calls and node class names that occur under `stmt`."""
    from tvm import tir
    from tvm.tir import stmt_functor
    calls, nodes = set(), set()

    def visit(node):
        nodes.add(type(node).__name__)
        if isinstance(node, tir.Call):
            calls.add(str(getattr(node.op, "name", node.op)))

    stmt_functor.post_order_visit(stmt, visit)
    return calls, nodes


def _store_of(block):
    from tvm import tir
    from tvm.tir import stmt_functor
    found = []

    def visit(node):
        if isinstance(node, tir.BufferStore):
            found.append(node)

    stmt_functor.post_order_visit(block.body, visit)
    return found


def _strip_cast(expr):
    from tvm import tir
    while isinstance(expr, tir.Cast):
        expr = expr.value
    return expr


def spec_from_prim_func(func, name):
    """PrimFunc -> OpSpec.  Raises UnsupportedWorkload for anything outside the five classes."""
    from tvm import tir

    params = [func.buffer_map[p] for p in func.params if p in func.buffer_map]
    if len(params) < 2:
        raise UnsupportedWorkload(f"{name}: expected at least one input and one output buffer")
    out = params[-1]
    ins = params[:-1]
    blocks = _collect_blocks(func)
    if not blocks:
        raise UnsupportedWorkload(f"{name}: no compute blocks")
    red = [b for b in blocks if b.has_reduce]
    upper = None
    if func.attrs is not None and "tir_var_upper_bound" in func.attrs:
        bounds = func.attrs["tir_var_upper_bound"]
        vals = [int(v) for v in bounds.values()]
        upper = max(vals) if vals else None

    def last_dim(buf):
        d = _static(buf.shape[-1])
        if d is None:
            raise UnsupportedWorkload(f"{name}: the innermost dim of {buf.name} must be static")
        return d

    if not red:
        if len(blocks) != 1:
            raise UnsupportedWorkload(f"{name}: elementwise functions must be a single block")
        stores = _store_of(blocks[0].block)
        if len(stores) != 1:
            raise UnsupportedWorkload(f"{name}: expected one store")
        value = stores[0].value
        h = last_dim(out)
        if isinstance(value, tir.Cast) and isinstance(value.value, tir.BufferLoad) and len(ins) == 1:
            return OpSpec(name, "cast", str(ins[0].dtype), str(out.dtype), cols=h, upper=upper)
        if isinstance(value, tir.Add) and isinstance(value.a, tir.BufferLoad) and isinstance(value.b, tir.BufferLoad) \
                and len(ins) == 2:
            return OpSpec(name, "add", str(ins[0].dtype), str(out.dtype), cols=h, upper=upper)
        if isinstance(value, tir.BufferLoad) and len(ins) == 1 and str(ins[0].dtype) == str(out.dtype):
            return OpSpec(name, "copy", str(ins[0].dtype), str(out.dtype), cols=h, upper=upper)
        raise UnsupportedWorkload(f"{name}: unrecognised elementwise expression {value}")

    first = red[0]
    stores = _store_of(first.block)
    # matmul: the reduction block accumulates a product of loads from two different inputs
    for st in stores:
        v = st.value
        if isinstance(v, tir.Add):
            prod = v.b if isinstance(_strip_cast(v.b), tir.Mul) else v.a
            prod = _strip_cast(prod)
            if isinstance(prod, tir.Mul):
                a, b = _strip_cast(prod.a), _strip_cast(prod.b)
                if isinstance(a, tir.BufferLoad) and isinstance(b, tir.BufferLoad) and \
                        not a.buffer.same_as(b.buffer):
                    w = ins[1]
                    if len(w.shape) != 2:
                        raise UnsupportedWorkload(f"{name}: weight must be [N, K]")
                    n, k = _static(w.shape[0]), _static(w.shape[1])
                    if n is None or k is None or last_dim(ins[0]) != k or last_dim(out) != n:
                        raise UnsupportedWorkload(f"{name}: only the NT layout X[m,K].W[N,K]^T is supported")
                    rows = [_static(d) for d in ins[0].shape[:-1]]
                    dynamic = any(d is None for d in rows)
                    # what follows the weight: an optional bias [N], then residuals shaped like the output
                    # (fused_NT_matmul2_add1_add3_add3, experiment/ModelIR/dolly-v2-3b-q0f16/before_dl.py:163)
                    extra = list(ins[2:])
                    bias = bool(extra) and len(extra[0].shape) == 1
                    if bias and _static(extra[0].shape[0]) != n:
                        raise UnsupportedWorkload(f"{name}: bias must have N = {n} elements")
                    res = extra[1:] if bias else extra
                    if len(res) > 2 or any(len(r.shape) != len(out.shape) or _static(r.shape[-1]) != n for r in res):
                        raise UnsupportedWorkload(f"{name}: at most two residuals shaped like the output are supported")
                    calls, _ = _calls_and_ops(func.body)
                    act = "gelu" if any("erf" in c for c in calls) else ""
                    unknown = [c for c in calls if not any(t in c for t in ("erf", "if_then_else", "likely"))]
                    if unknown:
                        raise UnsupportedWorkload(f"{name}: matmul tail calls {sorted(unknown)} have no fused kernel")
                    if str(out.dtype) not in ("float16", "float32"):
                        raise UnsupportedWorkload(f"{name}: output dtype {out.dtype}")
                    kw = dict(cols=n, k=k, bias=bias, residuals=len(res), act=act)
                    if not dynamic and all(d == 1 for d in rows):
                        return OpSpec(name, "gemv", "float16", str(out.dtype), upper=1, **kw)
                    return OpSpec(name, "gemm", "float16", str(out.dtype), upper=upper, **kw)
    # general reduction over the last dim
    calls, nodes = _calls_and_ops(func.body)
    if any("exp" in c for c in calls) and "Max" in nodes and _static(ins[0].shape[-1]) is None:
        # softmax over a symbolic last dim (the attention scores [1, heads, n, m] of
        # experiment/ModelIR/dolly-v2-3b-q0f16/before_dl.py:756-800): cols = 0 means "read it from the tensor"
        return OpSpec(name, "softmax", str(ins[0].dtype), str(out.dtype), cols=0, upper=upper)
    h = last_dim(ins[0])
    eps = 0.0
    from tvm.tir import stmt_functor
    consts = []
    stmt_functor.post_order_visit(func.body, lambda nd: consts.append(float(nd.value)) if isinstance(nd, tir.FloatImm) else None)
    small = [c for c in consts if 0.0 < c < 1e-3 and abs(c - 1.0 / h) > 1e-9 * (1.0 / h) + 1e-12]
    if small:
        eps = min(small)
    if any("exp" in c for c in calls) and "Max" in nodes:
        return OpSpec(name, "softmax", str(ins[0].dtype), str(out.dtype), cols=h, upper=upper)
    if any("rsqrt" in c for c in calls):
        n_red_outputs = len(stores)
        if n_red_outputs >= 2 and len(ins) == 3:
            return OpSpec(name, "layer_norm", str(ins[0].dtype), str(out.dtype), cols=h, eps=eps, upper=upper)
        if n_red_outputs == 1 and len(ins) == 2:
            return OpSpec(name, "rms_norm", str(ins[0].dtype), str(out.dtype), cols=h, eps=eps, upper=upper)
    raise UnsupportedWorkload(f"{name}: reduction pattern not recognised (calls {sorted(calls)})")


class FuncInfo:
    """Kind, dynamic arguments and kernel binding of one workload function."""

    def __init__(self, func, name="main"):
        self.name = name
        self.func = func
        if isinstance(func, OpSpec):
            self.spec = func
            self.dynamic_args = [] if func.op == "gemv" else ["n"]
        elif isinstance(func, dict):
            self.spec = OpSpec.from_dict(func)
            self.dynamic_args = [] if self.spec.op == "gemv" else ["n"]
        else:
            self.spec = spec_from_prim_func(func, name)
            self.dynamic_args = self._dynamic_args(func)
        # for each dynamic argument: "rows" (it multiplies the row count) or "cols" (it is the reduced,
        # innermost dim, as in a softmax over a symbolic length)
        self.dynamic_roles = self._dynamic_roles(func) if not isinstance(func, (OpSpec, dict)) else ["rows"] * len(self.dynamic_args)
        self.static_rows = self._static_rows(func) if not isinstance(func, (OpSpec, dict)) else 1
        self.kind = _KIND_OF[self.spec.kind]
        self.use_fp16 = "float16" in (self.spec.in_dtype, self.spec.out_dtype)
        self.in_dtype = self.spec.in_dtype
        self.out_dtype = self.spec.out_dtype

    @staticmethod
    def _dynamic_args(func):
        dyn = []
        for p in func.params:
            if p not in func.buffer_map:
                continue
            for dim in func.buffer_map[p].shape:
                if _static(dim) is None and not any(dim.same_as(d) for d in dyn):
                    if len(dyn) < 2:
                        dyn.append(dim)
                    else:
                        raise UnsupportedWorkload("at most two dynamic shape dimensions are supported")
        return [getattr(d, "name", str(d)) for d in dyn]

    def _dynamic_roles(self, func):
        first = func.buffer_map[[p for p in func.params if p in func.buffer_map][0]]
        last = first.shape[-1]
        roles = []
        for name in self.dynamic_args:
            is_last = _static(last) is None and getattr(last, "name", str(last)) == name
            roles.append("cols" if is_last else "rows")
        return roles

    @staticmethod
    def _static_rows(func):
        """Product of the static dims of the first input that are not its innermost one."""
        first = func.buffer_map[[p for p in func.params if p in func.buffer_map][0]]
        rows = 1
        for d in first.shape[:-1]:
            v = _static(d)
            if v is not None:
                rows *= v
        return rows

    def __repr__(self):
        return f'FuncInfo("{self.name}", {self.kind.name}, {self.spec})'
