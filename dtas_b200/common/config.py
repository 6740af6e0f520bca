"""Dispatch vocabulary: ranges of the symbolic dim and per-class kernel configurations.

`Range` and `generate_range_list` keep the reference's semantics
(python/dtas/common/config.py:21-78): closed integer ranges of width `div_factor` starting at
1, a name suffix `_n_1_to_256_`, and `merge` for adjacent ranges that picked the same
configuration.  The Config classes name the knobs of the hand-written kernels instead of TIR
schedule knobs; equality and hashing go through `to_dict`, as in the reference
(python/dtas/common/config.py:96-127).
"""
from typing import List


class Range:
    def __init__(self, var, start: int, end: int) -> None:
        self.var = var if isinstance(var, str) else getattr(var, "name", str(var))
        self.start = int(start)
        self.end = int(end)
        self.tuned = False

    def to_suffix(self):
        return "_" + self.var + "_" + str(self.start) + "_to_" + str(self.end) + "_"

    def merge(self, other: "Range") -> "Range":
        if self.var != other.var:
            raise ValueError("can not merge different var")
        if self.end == other.start - 1:
            return Range(self.var, self.start, other.end)
        if self.start == other.end + 1:
            return Range(self.var, other.start, self.end)
        raise ValueError("can not merge non-adjacent ranges")

    def __contains__(self, value):
        return self.start <= value <= self.end

    def __repr__(self) -> str:
        return f"<{self.var}: Range({self.start}, {self.end})>"

    __str__ = __repr__

    def __eq__(self, o) -> bool:
        return isinstance(o, Range) and (self.var, self.start, self.end) == (o.var, o.start, o.end)

    def __hash__(self) -> int:
        return hash((self.var, self.start, self.end))


def generate_range_list(var, start: int, end: int, div_factor: int) -> List[Range]:
    assert start < end
    assert div_factor > 0
    if end - start <= div_factor:
        return [Range(var, start, start + div_factor - 1)]
    ranges = []
    while start < end:
        ranges.append(Range(var, start, start + div_factor - 1))
        start += div_factor
    return ranges


class Config:
    """Base of the per-class configurations; hash / eq by content."""

    kind = "fallback"

    def to_dict(self):
        return dict(self.__dict__, kind=self.kind)

    @classmethod
    def from_dict(cls, d):
        d = dict(d)
        kind = d.pop("kind", cls.kind)
        klass = {c.kind: c for c in (ElementwiseConfig, ReductionConfig, GEMVConfig, GEMMConfig)}.get(kind, cls)
        obj = klass.__new__(klass)
        obj.__dict__.update(d)
        return obj

    def __eq__(self, other):
        return isinstance(other, Config) and self.to_dict() == other.to_dict()

    def __hash__(self):
        return hash(tuple(sorted((k, str(v)) for k, v in self.to_dict().items())))

    def __repr__(self):
        return f"{type(self).__name__}({self.to_dict()})"


class ElementwiseConfig(Config):
    """16-byte vectors, `unroll` vectors in flight per thread, 256 threads, grid capped at
    `ctas_per_sm` x SMs (reference knobs: len_tx, vector_size, grid_size, unroll_depth;
    python/dtas/common/config.py:407-429)."""
    kind = "elementwise"

    def __init__(self, variant: str):
        self.variant = variant
        self.len_tx = 256
        self.vector_bytes = 16
        self.unroll = int(variant.rsplit("unroll", 1)[1]) if "unroll" in variant else 1


class ReductionConfig(Config):
    """Threads per row and register chunks per thread (reference knobs: len_tx, bx_factor,
    temp_storage, vector_size; python/dtas/common/config.py:130-190)."""
    kind = "reduction"

    def __init__(self, variant: str):
        self.variant = variant
        self.temp_storage = "generic" if "generic" in variant else "local"


class GEMVConfig(Config):
    """Warps per output row and 16-byte loads in flight per lane (reference knobs: TS, TR,
    TILE_S, TILE_R, VEC_LOAD, VEC_C; python/dtas/common/config.py:338-374)."""
    kind = "gemv"

    def __init__(self, variant: str):
        self.variant = variant


class GEMMConfig(Config):
    """tcgen05 tile (128 x BN x 64), pipeline stages and split-K factor (reference knobs:
    i, j, micro_shape_x/y/k, in_vec_len, ...; python/dtas/common/config.py:193-294)."""
    kind = "gemm"

    def __init__(self, variant: str):
        self.variant = variant


def config_for(kind: str, variant: str) -> Config:
    return {"elementwise": ElementwiseConfig, "reduction": ReductionConfig, "gemv": GEMVConfig,
            "gemm": GEMMConfig}[kind](variant)
