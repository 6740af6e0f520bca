"""dtas_b200: sm_100a kernels behind the DTAS (JackWeiw/dtas) Python surface.

Mirrors the reference package surface (python/dtas/__init__.py:1-8): `arch`, `Config`,
`get_log_level` / `set_log_level`; plus the entry points `Engine`
(python/dtas/engine/tuner.py:22) and `load_module_from_file`
(python/dtas/codegen/runtime_packer.py:260).
"""
from .logging import get_log_level, set_log_level  # noqa: F401
from . import arch  # noqa: F401,E402
from .common.config import Config  # noqa: F401,E402
from .engine.tuner import Engine  # noqa: F401,E402
from .codegen.runtime_packer import load_module_from_file  # noqa: F401,E402
