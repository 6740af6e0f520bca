"""Generates the fixtures that pin parity to the reference's own PrimFunc text.

    python tests/golden/make_ref_golden.py [--ref <reference tree>] [key ...]

For every entry of ref_cases.SOURCES this script
  1. opens the reference file and cuts out the source of its `@I.ir_module class Module`
     (the `@R.function` members are dropped: Relax functions are not kernels, and the rest of
     the file imports the reference package, which needs a TVM this image does not have);
  2. parses that text with the TVM at hand (the fork bundled with tilelang) - the TVMScript
     parser reads source through `inspect`, so the text goes through a temporary .py file that
     is deleted afterwards; nothing of it is written into this repository;
  3. builds the PrimFuncs for target "c" (g++ -O2 -mf16c -Dhalf=_Float16) and runs them on the
     seeded inputs of ref_cases.make_inputs for n in {1, 17, 256, 257, 1025};
  4. writes
       ref_<key>.npz            kept output rows per n (`n<n>`) and their indices (`n<n>_rows`)
       ref_modules/<key>.json   the parsed IRModule (tvm.ir.save_json), which the GPU tests hand to
                                Engine.tune_module - the reference tree itself does not travel
       ref_golden_meta.json     per key: reference file, line span and SHA-256 of the module text,
                                PrimFunc name; per n: CRC-32 of the inputs, shape, dtype and SHA-256
                                of the whole output.
The generator is a TVM build of the reference's PrimFuncs for the CPU, not the author's own
CUDA build of them (that TVM is neither vendored nor pinned by the reference).
"""
import argparse
import hashlib
import importlib.util
import json
import os
import re
import shutil
import sys
import tempfile
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from tests.golden.ref_cases import SOURCES, make_inputs, n_values, stored_rows  # noqa: E402

PRELUDE = "import tilelang\nfrom tilelang import tvm\nfrom tvm.script import ir as I, tir as T\n"
CC_OPTIONS = ["-O2", "-mf16c", "-Dhalf=_Float16"]


def module_text(path):
    """(text of the `Module` class without Relax members, (first line, last line)) of a reference file.
    Simple top-level assignments above the class (`dtype = "float16"`) are kept: the class reads them."""
    with open(path) as f:
        lines = f.read().split("\n")
    start = next(i for i, ln in enumerate(lines) if ln.startswith("@I.ir_module"))
    pre = [ln for ln in lines[:start] if re.match(r'^\w+\s*=\s*["\d]', ln)]
    end = start + 2
    while end < len(lines) and (lines[end].strip() == "" or lines[end][0] in " \t#"):
        end += 1
    kept, in_relax = [], False
    for ln in lines[start:end]:
        if re.match(r"^    @R\.function", ln):
            in_relax = True
            continue
        if re.match(r"^    @T\.prim_func", ln):
            in_relax = False
        if not in_relax:
            kept.append(ln)
    while kept and kept[-1].strip() == "":
        kept.pop()
    return "\n".join(pre + kept) + "\n", (start + 1, end)


def parse_module(text, tag):
    """Executes the module text under the TVM of this image and returns the IRModule."""
    tmp = tempfile.mkdtemp(prefix="dtas_ref_")
    try:
        src = os.path.join(tmp, f"refmod_{tag}.py")
        with open(src, "w") as f:
            f.write(PRELUDE + text)
        spec = importlib.util.spec_from_file_location(f"refmod_{tag}", src)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = mod
        spec.loader.exec_module(mod)
        return mod.Module
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def build_for_cpu(tvm, ir_mod):
    """IRModule -> loaded runtime module; private PrimFuncs get their name as global symbol."""
    funcs = {gv.name_hint: fn.with_attr("global_symbol", gv.name_hint) for gv, fn in ir_mod.functions.items()}
    mod = tvm.IRModule(funcs)
    lib = tvm.build(mod, target="c") if hasattr(tvm, "build") else tvm.compile(mod, target="c")
    tmp = tempfile.mkdtemp(prefix="dtas_ref_")
    path = os.path.join(tmp, "ref.so")
    lib.export_library(path, options=CC_OPTIONS)
    return tvm.runtime.load_module(path), tmp


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("DTAS_REFERENCE_TREE") or os.path.join(HERE, "..", "..", "..", "reference"),
                    help="checkout of the reference; default: $DTAS_REFERENCE_TREE, else `reference` beside this repository")
    ap.add_argument("keys", nargs="*")
    args = ap.parse_args()
    import tilelang  # noqa: F401
    from tilelang import tvm
    to_nd = tvm.runtime.tensor if hasattr(tvm.runtime, "tensor") else tvm.nd.array

    meta_path = os.path.join(HERE, "ref_golden_meta.json")
    meta = {}
    if args.keys and os.path.exists(meta_path):
        with open(meta_path) as f:
            meta = json.load(f)
    os.makedirs(os.path.join(HERE, "ref_modules"), exist_ok=True)
    for key, src in SOURCES.items():
        if args.keys and key not in args.keys:
            continue
        text, span = module_text(os.path.join(args.ref, src["path"]))
        ir_mod = parse_module(text, key)
        with open(os.path.join(HERE, "ref_modules", f"{key}.json"), "w") as f:
            f.write(tvm.ir.save_json(ir_mod))
        rt, tmp = build_for_cpu(tvm, ir_mod)
        arrays, cases = {}, {}
        for n in n_values(key):
            ins, out = make_inputs(key, n)
            nds = [to_nd(a) for a in ins] + [to_nd(out)]
            rt[src["func"]](*nds)
            res = nds[-1].numpy()
            flat = res.reshape(-1, res.shape[-1])
            rows = stored_rows(key, flat.shape[0])
            arrays[f"n{n}"] = flat[rows]
            arrays[f"n{n}_rows"] = np.asarray(rows, np.int64)
            cases[str(n)] = {
                "input_crc32": [zlib.crc32(np.ascontiguousarray(a).tobytes()) for a in ins],
                "shape": list(res.shape), "dtype": str(res.dtype),
                "output_sha256": hashlib.sha256(np.ascontiguousarray(res).tobytes()).hexdigest(),
            }
            print(key, n, res.shape, res.dtype, f"{len(rows)} rows kept")
        shutil.rmtree(tmp, ignore_errors=True)
        np.savez_compressed(os.path.join(HERE, f"ref_{key}.npz"), **arrays)
        meta[key] = {"source": src["path"], "lines": list(span), "func": src["func"],
                     "module_text_sha256": hashlib.sha256(text.encode()).hexdigest(), "cases": cases}
    meta["_generator"] = {"tvm": tvm.__version__, "target": "c", "cc_options": CC_OPTIONS}
    with open(meta_path, "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)


if __name__ == "__main__":
    main()
