"""Workload descriptions accepted by Engine.tune_module.

Two equivalent forms:
  * a TVM IRModule of TVMScript PrimFuncs, as in the reference's tuning_test/*.py
    (builders in .tir_defs; needs an importable `tvm`), or
  * a dict / list of OpSpec, the same information without TVM.
"""
from .spec import OpSpec, default_module, llama2_7b_specs  # noqa: F401
