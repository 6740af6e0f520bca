"""CPU checker for the dtas_b200 kernels.  TEST INFRASTRUCTURE, not product.

Only tests/, __graft_entry__.smoke() and the cpu_baseline / --impl reference legs of
bench.py may import this package; nothing under dtas_b200/ does.
"""
from .cpu_oracle import *  # noqa: F401,F403
