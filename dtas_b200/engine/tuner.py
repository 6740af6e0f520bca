"""Engine: the entry point of the library, same call shape as the reference.

    Engine(topk, parallel_build, work_dir).tune_module(mod, arch, range_div_factor) -> runtime module

In the reference this runs a search: per PrimFunc and per range of the symbolic dim it asks a
policy for top-k schedule candidates, builds and times each with TVM, keeps the best, merges
neighbouring ranges that chose the same config and emits the index table of the generated
host code (python/dtas/engine/tuner.py:26-51, 53-133, 135-154, 156-209, 211-299).

Here the kernels are hand-written and the choice per call shape is made inside the library
(ew_cfg / row_cfg / pick_wpr / plan_gemm in dtas_b200/csrc), so nothing is built or timed:
`tune_module` classifies each function, walks the same ranges, asks the library which kernel
variant each range dispatches to, merges equal neighbours exactly as the reference does, and
returns a runtime module whose functions call the C ABI.  `topk` and `parallel_build` are
accepted for compatibility and unused.  The bucket index is min((m - 1) / width, last): the
reference's `n / 256` sends n = 256 to the second bucket (tuner.py:171-174), which is not
reproduced.
"""
import json
import os
from typing import Dict, List, Tuple

from .. import _abi
from ..codegen.runtime_packer import MODULE_FILE, RuntimeModule
from ..common.analysis import FuncInfo, UnsupportedWorkload
from ..common.config import Config, Range, config_for, generate_range_list
from ..logging import debug_info, get_log_level
from ..workloads.spec import OpSpec

DEFAULT_UPPER_BOUND = 2048   # the reference's default when no tir_var_upper_bound is given


class Engine:
    def __init__(self, topk: int = 10, parallel_build: bool = True, work_dir: str = None) -> None:
        self.topk = topk
        self.parallel_build = parallel_build
        self.work_dir = work_dir
        self.upper_bound: Dict[str, int] = {}
        if work_dir is not None:
            os.makedirs(work_dir, exist_ok=True)

    # -- module handling -------------------------------------------------------------------
    @staticmethod
    def _functions(mod) -> List[Tuple[str, object]]:
        """(name, PrimFunc | OpSpec) pairs of an IRModule, a dict, a list of OpSpec or one OpSpec."""
        if isinstance(mod, OpSpec):
            return [(mod.name, mod)]
        if isinstance(mod, (list, tuple)):
            return [(s.name, s) for s in mod]
        if isinstance(mod, dict):
            return list(mod.items())
        if hasattr(mod, "functions"):      # tvm.IRModule; Relax functions are not kernels
            out = []
            for gv, func in mod.functions.items():
                if type(func).__name__ == "PrimFunc":
                    out.append((gv.name_hint, func))
            return out
        raise TypeError(f"cannot read functions from {type(mod).__name__}")

    def _collect_upper_bounds(self, mod):
        """`tir_var_upper_bound` may sit on any function of the module (tuner.py:62-65)."""
        if not hasattr(mod, "functions"):
            return
        for _, func in mod.functions.items():
            if func.attrs is not None and "tir_var_upper_bound" in func.attrs:
                for k, v in func.attrs["tir_var_upper_bound"].items():
                    self.upper_bound[str(k)] = int(v)

    # -- ranges ----------------------------------------------------------------------------
    def gen_range_tuples(self, func_info: FuncInfo, range_div_factor: int):
        """One tuple of Ranges per bucket: the cartesian product of the range lists of up to two symbolic
        dims, the first dim slowest (python/dtas/engine/tuner.py:135-154)."""
        if len(func_info.dynamic_args) == 0:
            return [()]
        import itertools
        range_lists = []
        for dyn in func_info.dynamic_args:
            upper = func_info.spec.upper or self.upper_bound.get(dyn) or DEFAULT_UPPER_BOUND
            self.upper_bound[dyn] = upper
            range_lists.append(generate_range_list(dyn, 1, upper, range_div_factor))
        if len(range_lists) > 2:
            raise UnsupportedWorkload("at most two symbolic dims are supported")
        return [tuple(rt) for rt in itertools.product(*range_lists)]

    @staticmethod
    def merge_same_configs(range_to_config: Dict[Tuple[Range], Config]) -> Dict[Tuple[Range], Config]:
        """Adjacent ranges with equal configs collapse into one (tuner.py:211-299)."""
        merged: List[Tuple[Tuple[Range], Config]] = []
        for rt, cfg in range_to_config.items():
            if merged and len(rt) == 1 and merged[-1][1] == cfg:
                prev = merged[-1][0][0]
                merged[-1] = ((prev.merge(rt[0]),), cfg)
            else:
                merged.append((rt, cfg))
        return dict(merged)

    def get_index_table(self, merged: Dict[Tuple[Range], Config], range_div_factor: int):
        """index_table[i] = position in `merged` of the config serving bucket i, plus the statement(s)
        that compute the bucket index from the dynamic dim(s) (tuner.py:156-209).  With two symbolic dims
        the table is row-major over (bucket of the first dim, bucket of the second)."""
        items = list(merged.items())
        if not items or len(items[0][0]) == 0:
            return [], ""
        width = range_div_factor
        if len(items[0][0]) == 1:
            name = items[0][0][0].var
            table = []
            for i, (rt, _) in enumerate(items):
                table += [i] * len(range(rt[0].start, rt[0].end + 1, width))
            last = len(table) - 1
            return table, f"int64_t index = (({name} - 1)/{width}) > {last} ? {last} : ({name} - 1)/{width};"
        # two dims: nothing was merged, one entry per (bucket, bucket)
        n0 = len({rt[0].start for rt, _ in items})
        n1 = len({rt[1].start for rt, _ in items})
        v0, v1 = items[0][0][0].var, items[0][0][1].var
        table = list(range(len(items)))
        stmt = (f"int64_t i0 = (({v0} - 1)/{width}) > {n0 - 1} ? {n0 - 1} : ({v0} - 1)/{width}; "
                f"int64_t i1 = (({v1} - 1)/{width}) > {n1 - 1} ? {n1 - 1} : ({v1} - 1)/{width}; "
                f"int64_t index = i0 * {n1} + i1;")
        return table, stmt

    # -- per function ------------------------------------------------------------------------
    def tune_func(self, func, name: str, arch, range_div_factor: int):
        info = FuncInfo(func, name)
        spec = info.spec
        if get_log_level() >= 2:
            debug_info(f"{name}: {info.kind.name} {spec}")
        range_to_config: Dict[Tuple[Range], Config] = {}
        for rt in self.gen_range_tuples(info, range_div_factor):
            # the call shape at the upper end of the bucket: symbolic row dims multiply the static rows, a
            # symbolic innermost dim (softmax over a symbolic length) is the row length
            rows, cols = info.static_rows, spec.cols
            for r, role in zip(rt, info.dynamic_roles):
                if role == "cols":
                    cols = r.end
                else:
                    rows *= r.end
            variant = _abi.variant_of(spec.op, max(1, rows), cols or 1024, spec.k, getattr(arch, "dev_id", -1))
            range_to_config[rt] = config_for(spec.kind, variant)
        merged = self.merge_same_configs(range_to_config)
        table, stmt = self.get_index_table(merged, range_div_factor)
        return info, merged, table, stmt

    # -- on-device search (GEMM) -------------------------------------------------------------
    @staticmethod
    def gemm_candidates(m_hi: int):
        """(tile code, split) candidates for row counts up to m_hi; tile codes as in
        dtas_gemm_set_override (64/128/256 single-CTA widths, 512 two-CTA, 1024 swapped operands with a
        fixed split, 2048 swapped operands with stream-K, 4096 + width single-CTA tiles with stream-K,
        8192 + width K cut in two inside a two-CTA cluster, 16384 + S swapped operands with K cut in S
        inside a cluster)."""
        cands = []
        if m_hi <= 256:
            cands += [(1024, s) for s in (1, 2, 3, 4, 6, 8, 12, 16)] + [(2048, 0)]
            cands += [(bn, s) for bn in (64, 128, 256) for s in (1, 2, 4)] + [(bn, s) for bn in (64, 128) for s in (8, 16)]
            cands += [(4096 + bn, 0) for bn in (64, 128)]
            cands += [(8192 + 64, 0), (8192 + 128, 0)]
            if m_hi > 128:
                cands += [(512, 1), (513, 1)]     # a 256-row tile is at least half full
            if m_hi <= 64:
                cands += [(16384 + s, 0) for s in (2, 3, 4)]
        elif m_hi <= 1024:
            cands += [(bn, s) for bn in (128, 256) for s in (1, 2)] + [(64, s) for s in (1, 2, 4, 8)] + [(128, 4), (128, 8)]
            cands += [(512, 1), (513, 1), (4096 + 64, 0), (4096 + 128, 0), (4096 + 256, 0), (8192 + 64, 0), (8192 + 128, 0)]
        else:
            # above 1024 rows the two-CTA kernel wins whenever its 256 x 256 tiles fill the SM pairs; on
            # narrow column shards they do not (m = 4096, N = 512: 32 tiles on 74 pairs), and single-CTA
            # tiles, dealt out tile by tile or stream-K fashion, fill the machine instead
            cands += [(128, 1), (256, 1), (512, 1), (513, 1)]
        return cands

    def search_gemm(self, info: FuncInfo, ranges, device, samples=2, min_repeat_ms=5.0):
        """The reference's inner loop (python/dtas/schedule/tir_base.py:181-241: build each
        candidate, time it at sample shapes spread over the range, keep the fastest), with
        hand-written kernel variants as the candidates and CUDA-graph replay as the timer.
        Returns {range tuple: (GEMMConfig, tile code, split, mean us)}."""
        import torch
        from ..profiling import rotation_for, time_op
        from .. import ops
        lib = _abi.lib()
        spec = info.spec
        n, k = spec.cols, spec.k
        # enough copies of W that consecutive launches cannot be served from L2
        copies = rotation_for(2 * n * k, max_copies=8)
        ws = [(torch.randn((n, k), device=device, dtype=torch.float32) * 0.02).to(torch.float16) for _ in range(copies)]
        best = {}
        if not hasattr(self, "last_search_details"):
            self.last_search_details = []    # every candidate's time, for reports (retune --details)
        try:
            for rt in ranges:
                r = rt[0]
                ms = sorted({max(r.start, (r.start + r.end) // 2), r.end}) if samples >= 2 else [r.end]
                xs = [torch.randn((m, k), device=device, dtype=torch.float16) for m in ms]
                ys = [torch.empty((m, n), device=device, dtype=torch.float16) for m in ms]
                results = []
                for bn, split in self.gemm_candidates(r.end):
                    _abi.check(lib.dtas_gemm_set_override(bn, split))
                    variant = _abi.variant_of("gemm", r.end, n, k, device.index or 0)
                    total = 0.0
                    for x, y in zip(xs, ys):
                        t = time_op(lambda i: ops.gemm_nt(x, ws[i % copies], y), warmup=2, number=2, min_repeat_ms=min_repeat_ms, graph=True)
                        total += t["mean_us"]
                    results.append((total / len(xs), bn, split, variant))
                    if get_log_level() >= 2:
                        debug_info(f"{info.name} {r}: {variant} {total / len(xs):.2f} us")
                results.sort()
                us, bn, split, variant = results[0]
                best[rt] = (config_for("gemm", variant), bn, split, us)
                self.last_search_details.append({"n": n, "k": k, "m_lo": r.start, "m_hi": r.end, "sampled_m": ms,
                                                 "candidates": [{"us": round(u, 2), "bn": b, "split": sp, "variant": v}
                                                                for u, b, sp, v in results]})
                ops.poll_status(device.index or 0)
        finally:
            _abi.check(lib.dtas_gemm_set_override(0, 0))
        return best

    def tune_module(self, mod, arch, range_div_factor: int = 256, search: bool = False):
        """search=True (needs a GPU): GEMM functions are tuned on the device - every candidate
        kernel variant is timed per range, the winners are installed in the library's dispatch
        table and stored in work_dir, so `load_module_from_file` restores them."""
        self._collect_upper_bounds(mod)
        entries = {}
        for name, func in self._functions(mod):
            try:
                info, merged, table, stmt = self.tune_func(func, name, arch, range_div_factor)
                measured = None
                if search and info.spec.op == "gemm":
                    device = getattr(arch, "device", None)
                    if device is None:
                        raise RuntimeError("tune_module(search=True) needs a CUDA device")
                    ranges = self.gen_range_tuples(info, range_div_factor)
                    found = self.search_gemm(info, ranges, device)
                    merged = self.merge_same_configs({rt: cfg for rt, (cfg, _, _, _) in found.items()})
                    table, stmt = self.get_index_table(merged, range_div_factor)
                    measured = []
                    for rt, cfg in merged.items():
                        # tile code / split of any member range with this config
                        bn, split = next((b, s) for r2, (c2, b, s, _) in found.items() if c2 == cfg and r2[0].start >= rt[0].start and r2[0].end <= rt[0].end)
                        measured.append({"m_lo": rt[0].start, "m_hi": rt[0].end, "bn": bn, "split": split})
                        _abi.check(_abi.lib().dtas_gemm_table_set(info.spec.cols, info.spec.k, rt[0].start, rt[0].end, bn, split))
            except UnsupportedWorkload as e:
                if get_log_level() >= 1:
                    debug_info(f"skipping {name}: {e}")
                continue
            entries[name] = {
                "spec": info.spec.to_dict(),
                "kind": info.kind.name,
                "dynamic_args": info.dynamic_args,
                "range_div_factor": range_div_factor,
                "ranges": [({"start": rt[0].start, "end": rt[0].end, "suffix": rt[0].to_suffix(), "config": cfg.to_dict()}
                            if len(rt) == 1 else
                            {"start": [r.start for r in rt], "end": [r.end for r in rt],
                             "suffix": "_".join(r.to_suffix() for r in rt), "config": cfg.to_dict()})
                           if rt else {"config": cfg.to_dict()}
                           for rt, cfg in merged.items()],
                "index_table": table,
                "index_stmt": stmt,
            }
            if measured is not None:
                entries[name]["measured_table"] = measured
            if get_log_level() >= 1:
                debug_info(f"{name}: {info.kind.name}, {len(merged)} merged range(s)")
        record = {"library": _abi.lib().dtas_version().decode(), "arch": type(arch).__name__, "functions": entries}
        if self.work_dir is not None:
            with open(os.path.join(self.work_dir, MODULE_FILE), "w") as f:
                json.dump(record, f, indent=1)
        return RuntimeModule(record)
