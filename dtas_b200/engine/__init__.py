from .tuner import Engine  # noqa: F401
