"""Loads oracle/_ref/dtas_ref_primfuncs.so (the PrimFuncs built by TVM, see build_ref.py) and
calls its functions on numpy arrays.  TEST / BASELINE INFRASTRUCTURE, not product."""
import os

from .build_ref import REF_SO

_state = {}


def available():
    """(ok, why): the TVM runtime must import and the prebuilt library must exist."""
    if "ok" in _state:
        return _state["ok"], _state["why"]
    ok, why = True, ""
    if not os.path.exists(REF_SO):
        ok, why = False, f"{REF_SO} has not been built"
    else:
        try:
            from dtas_b200.workloads import tir_defs as td
            tvm = td._tvm()
            _state["tvm"] = tvm
            _state["mod"] = tvm.runtime.load_module(REF_SO)
        except Exception as e:  # noqa: BLE001 - any failure means "use the C port instead"
            ok, why = False, f"TVM runtime unavailable: {type(e).__name__}: {e}"
    _state["ok"], _state["why"] = ok, why
    return ok, why


def call(name, *arrays):
    """Runs PrimFunc `name` on numpy arrays (inputs then the output, updated in place is NOT
    guaranteed: the result array is returned)."""
    ok, why = available()
    if not ok:
        raise RuntimeError(why)
    tvm = _state["tvm"]
    to_nd = tvm.runtime.tensor if hasattr(tvm.runtime, "tensor") else tvm.nd.array
    nds = [to_nd(a) for a in arrays]
    _state["mod"][name](*nds)
    return nds[-1].numpy()


def prepare(name, *arrays):
    """-> zero-argument callable that re-runs the PrimFunc on pre-converted tensors (for timing)."""
    ok, why = available()
    if not ok:
        raise RuntimeError(why)
    tvm = _state["tvm"]
    to_nd = tvm.runtime.tensor if hasattr(tvm.runtime, "tensor") else tvm.nd.array
    nds = [to_nd(a) for a in arrays]
    fn = _state["mod"][name]
    return lambda: fn(*nds)
