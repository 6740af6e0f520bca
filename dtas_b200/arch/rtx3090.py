"""The reference's only hardware record, kept as data so its published numbers can be put
next to B200 figures (python/dtas/arch/RTX3090.py:6-36).  No kernel in this library runs on it."""
from .arch_base import Arch


class RTX3090(Arch):
    def __init__(self, dev_id=0):
        super().__init__()
        self.reg_cap = 65536
        self.smem_cap = 99 * 1024
        self.num_sm = 82
        self.max_resident_threads_per_sm = 1536
        self.max_resident_blocks_per_sm = 16
        self.max_registers_per_sm = 64 * 1024
        self.max_registers_per_block = 64 * 1024
        self.max_smem_per_sm = 100 * 1024
        self.max_smem_per_block = 99 * 1024
        self.max_threads_per_block = 1024
        self.warp_size = 32
        self.sm_partition = 4
        self.transaction_size = [32, 128]
        self.l2_cache_size = 6 * 1024
        self.bandwidth = [849, 1954, 54480]
        self.processing_power = [29.28, 29.28, 0.458, 142]
        self.platform = "CUDA"
        self.compute_capability = "86"
        self.target = "nvidia/geforce-rtx-3090"
        self.dev_id = dev_id
