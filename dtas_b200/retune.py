"""Offline re-tuning of the GEMM dispatch table on the GPU at hand.

    python -m dtas_b200.retune --out dtas_b200/tables/b200_gemm.json            # Llama-2-7B shapes, 1/2/4/8-way shards
    python -m dtas_b200.retune --shape 4096x4096 --shape 5120x13824 --out my_table.json
    python -m dtas_b200.retune --shape 2560x2560 --merge-into dtas_b200/tables/b200_gemm.json --out dtas_b200/tables/b200_gemm.json

The reference tunes every PrimFunc of a model once, offline, and ships the per-range winners
inside the generated host code (python/dtas/engine/tuner.py:103-133, 211-299).  This is the
same step for the hand-written GEMM variants: for each weight shape (n, k) and each range of
row counts it times every candidate (tile code, split-K) with Engine.search_gemm, merges
neighbouring ranges that chose the same variant, and writes the table as JSON.  A table found
at dtas_b200/tables/b200_gemm.json is installed when the library is loaded (dtas_b200._abi.lib);
shapes it does not cover are planned by the built-in cost model.
"""
import argparse
import json
import os

# Row-count ranges: fine below 256 (where the best variant changes quickly), two per power of
# two above, open-ended above 4096 like the reference's clamped last bucket.
M_RANGES = [(1, 16), (17, 32), (33, 64), (65, 128), (129, 192), (193, 256), (257, 384), (385, 512), (513, 768),
            (769, 1024), (1025, 1536), (1537, 2048), (2049, 3072), (3073, 4096), (4097, 1 << 30)]
LLAMA2_7B = [(12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008)]


def default_shapes():
    shapes = []
    for n, k in LLAMA2_7B:
        for g in (1, 2, 4, 8):
            if n % g == 0 and (n // g, k) not in shapes:
                shapes.append((n // g, k))
    return shapes


def merge_tables(old, new):
    """Shapes of `old` that `new` does not re-measure, then every shape of `new`."""
    fresh = {(s["n"], s["k"]) for s in new}
    return [s for s in old if (s["n"], s["k"]) not in fresh] + list(new)


def main():
    import torch
    from . import _abi
    from .common.analysis import FuncInfo
    from .common.config import Range
    from .engine.tuner import Engine
    from .logging import set_log_level
    from .workloads.spec import OpSpec

    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", action="append", default=[], help="NxK (weight rows x reduction length); repeatable")
    ap.add_argument("--out", required=True)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--min-repeat-ms", type=float, default=10.0)
    ap.add_argument("--details", default=None, help="also write every candidate's time per range to this JSON file")
    ap.add_argument("--merge-into", default=None, help="an existing table: its shapes are kept, re-measured ones replaced")
    a = ap.parse_args()
    shapes = [tuple(int(v) for v in s.lower().split("x")) for s in a.shape] or default_shapes()
    set_log_level(0)
    dev = torch.device("cuda", a.device)
    torch.cuda.set_device(dev)
    _abi.check(_abi.lib().dtas_gemm_table_clear())      # tune against the cost model's blank slate
    eng = Engine(1, True, None)
    table = []
    for (n, k) in shapes:
        info = FuncInfo(OpSpec(f"gemm_n{n}_k{k}", "gemm", cols=n, k=k))
        # sample each range at its midpoint and its end (the open last range at 8192)
        ranges = [(Range("n", lo, min(hi, 8192)),) for lo, hi in M_RANGES]
        found = eng.search_gemm(info, ranges, dev, samples=2, min_repeat_ms=a.min_repeat_ms)
        rows = []
        for (lo, hi), rt in zip(M_RANGES, ranges):
            cfg, bn, split, us = found[rt]
            if rows and rows[-1]["variant"].split("_m")[0] == cfg.variant.split("_m")[0] and rows[-1]["bn"] == bn \
                    and rows[-1]["split"] == split:
                rows[-1]["m_hi"] = hi
                rows[-1]["us_at_end"] = round(us, 2)
            else:
                rows.append({"m_lo": lo, "m_hi": hi, "bn": bn, "split": split, "variant": cfg.variant, "us_at_end": round(us, 2)})
        for r in rows:
            print(f"n={n} k={k} m={r['m_lo']}..{r['m_hi']}: {r['variant']}  {r['us_at_end']} us", flush=True)
        table.append({"n": n, "k": k, "rows": rows})
    if a.merge_into:
        table = merge_tables(json.load(open(a.merge_into)).get("gemm", []), table)
    rec = {"device": torch.cuda.get_device_name(dev), "library": _abi.lib().dtas_version().decode(), "gemm": table}
    os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
    with open(a.out, "w") as f:
        json.dump(rec, f, indent=1)
    print(f"wrote {a.out}")
    if a.details:
        with open(a.details, "w") as f:
            json.dump(eng.last_search_details, f, indent=1)


if __name__ == "__main__":
    main()
