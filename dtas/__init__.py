"""Import alias: `dtas` resolves to `dtas_b200`, so scripts written against the reference keep
their import lines (tuning_test/tune_cast.py:35-36: `from dtas.engine.tuner import Engine`,
`from dtas.arch import RTX3090`; python/dtas/__init__.py:1-8 for the package surface).

Every submodule of the reference package that has a counterpart here is registered under its
reference name - including the reference's spelling `dtas.common.analisys` - and points at the
same module object as its `dtas_b200` name, so state (log level, library handle) is shared.
"""
import importlib
import sys

import dtas_b200 as _impl
from dtas_b200 import *  # noqa: F401,F403
from dtas_b200 import Config, Engine, arch, get_log_level, load_module_from_file, set_log_level  # noqa: F401

_SUBMODULES = {
    "arch": "arch", "arch.arch_base": "arch.arch_base", "arch.RTX3090": "arch.rtx3090", "arch.B200": "arch.b200",
    "engine": "engine", "engine.tuner": "engine.tuner",
    "codegen": "codegen", "codegen.runtime_packer": "codegen.runtime_packer",
    "common": "common", "common.config": "common.config", "common.analisys": "common.analysis",
    "common.analysis": "common.analysis",
    "logging": "logging", "reference": "reference",
}
for _ref_name, _here in _SUBMODULES.items():
    _mod = importlib.import_module(f"dtas_b200.{_here}")
    sys.modules[f"{__name__}.{_ref_name}"] = _mod
    if "." not in _ref_name:
        globals()[_ref_name] = _mod

__version__ = getattr(_impl, "__version__", "0")
