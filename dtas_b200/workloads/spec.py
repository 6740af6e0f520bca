"""TVM-free description of one workload function: which operator class it belongs to, its
dtypes and its static dims.  The symbolic dim (the reference's `n = T.int64()`,
tuning_test/tune_cast.py:12) is always the row count and is never stored here."""
from dataclasses import dataclass, field, asdict
from typing import Dict, List, Optional

# operator -> FuncKind of the reference's classifier (python/dtas/common/analisys.py:49-55)
OP_KIND = {
    "cast": "elementwise", "add": "elementwise", "copy": "elementwise",
    "rms_norm": "reduction", "softmax": "reduction", "layer_norm": "reduction",
    "gemv": "gemv", "gemm": "gemm",
}


@dataclass
class OpSpec:
    """One function of a module.

    name      : function name the runtime module exposes (`rt_mod[name]`)
    op        : "cast" | "add" | "copy" | "rms_norm" | "softmax" | "layer_norm" | "gemv" | "gemm"
    in_dtype  : dtype of the streamed input ("float16" | "float32" | "int8")
    out_dtype : dtype of the output
    cols      : static row length H for elementwise / reduction ops (0 for a softmax whose reduction
                length is symbolic too: it is read from the tensor at call time); N for gemv / gemm
    k         : reduction length K for gemv / gemm
    eps       : epsilon of the norm ops
    bias      : gemv / gemm take a bias argument
    residuals : gemv / gemm add this many [m, N] tensors after the activation (0, 1 or 2)
    act       : activation fused behind the bias: "" or "gelu"
    upper     : upper bound of the symbolic dim (the reference's tir_var_upper_bound)
    """
    name: str
    op: str
    in_dtype: str = "float16"
    out_dtype: str = "float16"
    cols: int = 0
    k: int = 0
    eps: float = 0.0
    bias: bool = False
    residuals: int = 0
    act: str = ""
    upper: Optional[int] = None
    attrs: Dict[str, str] = field(default_factory=dict)

    def __post_init__(self):
        if self.op not in OP_KIND:
            raise ValueError(f"unknown op '{self.op}'")
        if self.residuals not in (0, 1, 2) or self.act not in ("", "gelu"):
            raise ValueError(f"{self.name}: residuals must be 0..2 and act '' or 'gelu'")
        if (self.residuals or self.act) and self.op not in ("gemv", "gemm"):
            raise ValueError(f"{self.name}: only gemv / gemm take a fused tail")

    @property
    def kind(self):
        return OP_KIND[self.op]

    def to_dict(self):
        return asdict(self)

    @staticmethod
    def from_dict(d):
        return OpSpec(**d)


def default_module() -> List[OpSpec]:
    """The five BASELINE workload families at their Llama-2-7B sizes."""
    return llama2_7b_specs()


def llama2_7b_specs() -> List[OpSpec]:
    specs = [
        OpSpec("cast", "cast", "float32", "float16", cols=4096),
        OpSpec("add", "add", "float16", "float16", cols=11008),
        OpSpec("copy", "copy", "float16", "float16", cols=11008),
        OpSpec("rms_norm", "rms_norm", "float16", "float16", cols=4096, eps=1e-6),
        OpSpec("softmax", "softmax", "float16", "float16", cols=4096),
    ]
    for n, k in [(4096, 4096), (11008, 4096), (4096, 11008), (32000, 4096)]:
        specs.append(OpSpec(f"gemv_n{n}_k{k}", "gemv", cols=n, k=k))
    for n, k in [(12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008)]:
        specs.append(OpSpec(f"gemm_n{n}_k{k}", "gemm", cols=n, k=k))
    return specs
