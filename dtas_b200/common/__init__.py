from .config import Config, Range, generate_range_list  # noqa: F401
