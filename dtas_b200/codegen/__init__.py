from .runtime_packer import RuntimeModule, load_module_from_file  # noqa: F401
