"""Hardware record, same field list as the reference's Arch (python/dtas/arch/arch_base.py:2-27)."""


class Arch:
    def __init__(self) -> None:
        self.reg_cap = 0
        self.smem_cap = 0
        self.compute_max_core = 0
        self.num_sm = 0
        self.max_resident_threads_per_sm = 0
        self.max_resident_blocks_per_sm = 0
        self.max_registers_per_sm = 0
        self.max_registers_per_block = 0
        self.max_smem_per_sm = 0
        self.max_smem_per_block = 0
        self.max_threads_per_block = 0
        self.warp_size = 0
        self.sm_partition = 0
        self.transaction_size = [0, 0]
        # half, single, double, tensor-core TFLOP/s
        self.processing_power = [0, 0, 0, 0]
        # GB/s: global memory, L2 (, shared memory)
        self.bandwidth = [0, 0]
        self.l2_cache_size = 0
        self.device = None          # torch.device, or None when built without a GPU
        self.platform = "unknown"
        self.compute_capability = "unknown"
        self.target = None
