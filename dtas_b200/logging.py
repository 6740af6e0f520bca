"""Global verbosity switch and a caller-tagged print, as in python/dtas/logging.py:1-19."""
import inspect
import sys

_verbose = 1


def set_log_level(verbose):
    global _verbose
    _verbose = verbose


def get_log_level():
    return _verbose


def debug_info(message: str):
    frame = inspect.stack()[1]
    print(f"({frame[1]}:{frame[2]}):{message}", file=sys.stderr)
