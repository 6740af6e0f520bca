"""Calling the kernels from a TVM runtime (Relax VM or plain packed-function calls).

In the reference the tuned functions live inside a `tvm.runtime.Module` and a Relax program
reaches them through `R.call_tir` / the VM (tuning_test/tune_cast.py:24-32,
python/dtas/codegen/runtime_packer.py:237-258).  Here the kernels live in libdtas_b200.so, so
the bridge is the other way round: every function of a RuntimeModule is registered as a TVM
global function `"<prefix>.<name>"` with the same destination-passing signature
(inputs..., output), and a Relax program calls it with

    R.call_dps_packed("dtas_b200.cast", (x,), out_sinfo=R.Tensor((1, n, 4096), "float16"))

on a VM created on a CUDA device.  Tensors cross the boundary through DLPack without a copy;
the kernels run on the current torch stream, which is the default stream unless the caller
changed it - the same one a default TVM runtime uses.  Needs an importable `tvm` whose runtime
was built with CUDA (the fork bundled with tilelang is one); nothing else in dtas_b200 imports it.
"""
import torch

from .workloads.tir_defs import _tvm


def _as_torch(t):
    if isinstance(t, torch.Tensor):
        return t
    return torch.from_dlpack(t)


def register_module(rt_mod, prefix="dtas_b200", override=True):
    """Registers `<prefix>.<name>` for every function of `rt_mod` (a dtas_b200 RuntimeModule).
    Returns {function name: global function name}."""
    tvm = _tvm()
    names = {}
    for name in rt_mod.keys():
        op = rt_mod[name]

        def packed(*args, _op=op):
            _op(*[_as_torch(a) for a in args])

        full = f"{prefix}.{name}"
        tvm.register_global_func(full, packed, override=override)
        names[name] = full
    return names


def get_packed(name, prefix="dtas_b200"):
    """The registered TVM function, as a Relax VM would look it up."""
    return _tvm().get_global_func(f"{prefix}.{name}")
