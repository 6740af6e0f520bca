"""Host logic without a GPU: ranges, merging, index tables, classification, Engine round trip."""
import json
import os

import pytest

import dtas_b200
from dtas_b200 import Engine, arch, load_module_from_file
from dtas_b200.codegen.runtime_packer import MODULE_FILE
from dtas_b200.common.analysis import FuncInfo, FuncKind
from dtas_b200.common.config import Config, Range, config_for, generate_range_list
from dtas_b200.workloads import OpSpec, llama2_7b_specs


def test_range_semantics():
    r = generate_range_list("n", 1, 4096, 256)
    assert len(r) == 16 and r[0] == Range("n", 1, 256) and r[-1] == Range("n", 3841, 4096)
    assert r[0].to_suffix() == "_n_1_to_256_"
    assert generate_range_list("n", 1, 100, 256) == [Range("n", 1, 256)]
    merged = r[0].merge(r[1])
    assert merged == Range("n", 1, 512) and r[1].merge(r[0]) == merged
    with pytest.raises(ValueError):
        r[0].merge(r[2])
    with pytest.raises(ValueError):
        r[0].merge(Range("m", 257, 512))
    assert 256 in r[0] and 257 not in r[0]


def test_config_equality_and_roundtrip():
    a, b = config_for("gemm", "gemm_tcgen05_bm128_bn256_bk64_s4_splitk1"), config_for("gemm", "gemm_tcgen05_bm128_bn256_bk64_s4_splitk1")
    c = config_for("gemm", "gemm_tcgen05_bm128_bn128_bk64_s6_splitk2")
    assert a == b and hash(a) == hash(b) and a != c
    assert Config.from_dict(a.to_dict()) == a
    assert config_for("elementwise", "ew_vec16_unroll4").unroll == 4


def test_merge_and_index_table():
    e = Engine()
    ranges = generate_range_list("n", 1, 1024, 256)
    cfgs = [config_for("elementwise", v) for v in ("a_unroll1", "a_unroll2", "a_unroll2", "a_unroll4")]
    merged = e.merge_same_configs({(r,): c for r, c in zip(ranges, cfgs)})
    keys = [k[0] for k in merged]
    assert keys == [Range("n", 1, 256), Range("n", 257, 768), Range("n", 769, 1024)]
    table, stmt = e.get_index_table(merged, 256)
    assert table == [0, 1, 1, 2]
    assert "(n - 1)/256" in stmt and "> 3 ? 3" in stmt


def test_engine_on_specs_roundtrip(tmp_path):
    dtas_b200.set_log_level(0)
    eng = Engine(10, parallel_build=True, work_dir=str(tmp_path))
    rt = eng.tune_module(llama2_7b_specs(), arch=arch.B200(0), range_div_factor=256)
    names = set(rt.keys())
    assert {"cast", "add", "copy", "rms_norm", "softmax", "gemv_n32000_k4096", "gemm_n22016_k4096"} <= names
    rec = json.load(open(os.path.join(str(tmp_path), MODULE_FILE)))
    for name, ent in rec["functions"].items():
        table = ent["index_table"]
        if ent["kind"] == "kFunc_GEMV":
            assert table == [] and ent["dynamic_args"] == []
            continue
        # total over every bucket, monotone, and consistent with the merged ranges
        assert len(table) == 8 and table == sorted(table) and table[0] == 0 and table[-1] == len(ent["ranges"]) - 1
        starts = [r["start"] for r in ent["ranges"]]
        ends = [r["end"] for r in ent["ranges"]]
        assert starts[0] == 1 and ends[-1] == 2048 and all(s == e + 1 for s, e in zip(starts[1:], ends[:-1]))
    op = rt["cast"]
    assert op.bucket_index(1) == 0 and op.bucket_index(256) == 0 and op.bucket_index(10 ** 6) == op.entry["index_table"][-1]
    rt2 = load_module_from_file(str(tmp_path))
    assert set(rt2.keys()) == names and rt2["gemm_n22016_k4096"].spec.k == 4096
    with pytest.raises(FileNotFoundError):
        load_module_from_file(str(tmp_path / "nothing"))


def test_classification_of_specs():
    assert FuncInfo(OpSpec("f", "cast", "float32", "float16", cols=8)).kind == FuncKind.kFunc_Elementwise
    assert FuncInfo(OpSpec("f", "softmax", cols=8)).kind == FuncKind.kFunc_Reduction
    g = FuncInfo(OpSpec("f", "gemv", cols=8, k=8))
    assert g.kind == FuncKind.kFunc_GEMV and g.dynamic_args == []
    assert FuncInfo(OpSpec("f", "gemm", cols=8, k=8)).kind == FuncKind.kFunc_GEMM
    with pytest.raises(ValueError):
        OpSpec("f", "conv2d")


def test_classification_of_tvmscript_primfuncs():
    """The reference's workload style: TVMScript PrimFuncs with a symbolic row count."""
    td = pytest.importorskip("dtas_b200.workloads.tir_defs")
    try:
        td._tvm()
    except ImportError:
        pytest.skip("no TVM in this environment")
    cases = {
        "cast": (td.cast(2560, "float16", "float32"), "cast", FuncKind.kFunc_Elementwise),
        "add": (td.add(2560, "int8"), "add", FuncKind.kFunc_Elementwise),
        "copy": (td.copy(2560, "float32"), "copy", FuncKind.kFunc_Elementwise),
        "rms_norm": (td.rms_norm(4096, 1e-6), "rms_norm", FuncKind.kFunc_Reduction),
        "softmax": (td.softmax(4096, "float16"), "softmax", FuncKind.kFunc_Reduction),
        "layer_norm": (td.layer_norm(2560, "float32", 1e-5), "layer_norm", FuncKind.kFunc_Reduction),
        "gemm": (td.gemm_nt(12288, 4096), "gemm", FuncKind.kFunc_GEMM),
        "gemv": (td.gemv(4096, 11008), "gemv", FuncKind.kFunc_GEMV),
    }
    for name, (func, op, kind) in cases.items():
        info = FuncInfo(func, name)
        assert info.spec.op == op and info.kind == kind, (name, info)
        assert info.dynamic_args == ([] if op == "gemv" else ["n"])
    assert FuncInfo(cases["cast"][0], "cast").spec.in_dtype == "float16"
    assert FuncInfo(cases["add"][0], "add").spec.in_dtype == "int8"
    assert abs(FuncInfo(cases["rms_norm"][0], "r").spec.eps - 1e-6) < 1e-12
    assert abs(FuncInfo(cases["layer_norm"][0], "l").spec.eps - 1e-5) < 1e-11
    g = FuncInfo(cases["gemm"][0], "g").spec
    assert (g.cols, g.k) == (12288, 4096)
    # Engine accepts the IRModule itself and honours tir_var_upper_bound
    dtas_b200.set_log_level(0)
    mod = td.make_module({"cast": cases["cast"][0], "softmax": cases["softmax"][0]}, upper_bound=4096)
    rt = Engine(1, True, None).tune_module(mod, arch=arch.B200(0), range_div_factor=256)
    assert set(rt.keys()) == {"cast", "softmax"}
    assert len(rt.record["functions"]["cast"]["index_table"]) == 16


def test_classification_of_fused_matmul_forms():
    """The fused matmul functions of the reference's model IR (bias, GELU, residual adds, trailing
    cast; dynamic rows or the single decode row) map to gemm / gemv specs with a fused tail."""
    td = pytest.importorskip("dtas_b200.workloads.tir_defs")
    try:
        td._tvm()
    except ImportError:
        pytest.skip("no TVM in this environment")
    forms = [
        (dict(), ("gemm", True, 0, "", "float16")),                                   # fused_NT_matmul_add
        (dict(act="gelu"), ("gemm", True, 0, "gelu", "float16")),                     # fused_NT_matmul3_add2_gelu
        (dict(residuals=2), ("gemm", True, 2, "", "float16")),                        # ..._add1_add3_add3
        (dict(residuals=2, out_dtype="float32"), ("gemm", True, 2, "", "float32")),   # ..._add1_add3_add3_cast
        (dict(dynamic=False, residuals=2), ("gemv", True, 2, "", "float16")),         # fused_NT_matmul8_add5_add7_add7
        (dict(dynamic=False, act="gelu"), ("gemv", True, 0, "gelu", "float16")),      # fused_NT_matmul9_add6_gelu1
        (dict(bias=False, residuals=1), ("gemm", False, 1, "", "float16")),
    ]
    for kw, (op, bias, n_res, act, out) in forms:
        s = FuncInfo(td.matmul_fused(2560, 10240, **kw), "f").spec
        assert (s.op, s.bias, s.residuals, s.act, s.out_dtype, s.cols, s.k) == (op, bias, n_res, act, out, 2560, 10240), (kw, s)
    with pytest.raises(ValueError):
        OpSpec("f", "softmax", cols=8, act="gelu")
    # a module record with a fused function survives the JSON round trip
    dtas_b200.set_log_level(0)
    mod = td.make_module({"ffn_up": td.matmul_fused(10240, 2560, act="gelu"),
                          "attn_out": td.matmul_fused(2560, 2560, residuals=2, out_dtype="float32")}, upper_bound=1024)
    rt = Engine(1, True, None).tune_module(mod, arch=arch.B200(0), range_div_factor=256)
    assert rt["ffn_up"].spec.act == "gelu" and rt["attn_out"].spec.residuals == 2
    assert OpSpec.from_dict(rt.record["functions"]["attn_out"]["spec"]).out_dtype == "float32"


def test_classification_of_softmax_with_two_symbolic_dims():
    """fused_softmax_cast3 of the reference's model IR: [1, 32, n, m], softmax over the symbolic m."""
    td = pytest.importorskip("dtas_b200.workloads.tir_defs")
    try:
        td._tvm()
    except ImportError:
        pytest.skip("no TVM in this environment")
    info = FuncInfo(td.softmax_dynamic(32, "float32"), "attn_softmax")
    assert info.kind == FuncKind.kFunc_Reduction and info.spec.op == "softmax"
    assert (info.spec.cols, info.spec.in_dtype, info.spec.out_dtype) == (0, "float32", "float16")
    assert info.dynamic_args == ["n", "m"]
    dtas_b200.set_log_level(0)
    rt = Engine(1, True, None).tune_module(td.make_module({"attn_softmax": td.softmax_dynamic(32, "float32")}, upper_bound=2048),
                                           arch=arch.B200(0), range_div_factor=256)
    assert rt["attn_softmax"].spec.cols == 0
    # the range table is the cartesian product of the two dims' ranges, first dim slowest, as the
    # reference builds it (python/dtas/engine/tuner.py:135-154): 8 x 8 buckets of 256 up to 2048
    ent = rt.record["functions"]["attn_softmax"]
    assert info.dynamic_roles == ["rows", "cols"] and info.static_rows == 32
    assert len(ent["ranges"]) == 64 and ent["index_table"] == list(range(64))
    assert ent["ranges"][0]["start"] == [1, 1] and ent["ranges"][0]["end"] == [256, 256]
    assert ent["ranges"][9]["start"] == [257, 257] and ent["ranges"][63]["end"] == [2048, 2048]
    assert "i0 * 8 + i1" in ent["index_stmt"]
    op = rt["attn_softmax"]
    assert op.bucket_index(1, 1) == 0 and op.bucket_index(257, 300) == 9 and op.bucket_index(10 ** 6, 10 ** 6) == 63
    # the kernel layout follows the reduction length of the bucket, not a nominal one
    assert ent["ranges"][0]["config"] != ent["ranges"][7]["config"]
