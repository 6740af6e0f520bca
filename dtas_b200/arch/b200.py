"""NVIDIA B200 (sm_100a) record, the counterpart of python/dtas/arch/RTX3090.py:6-36."""
from .arch_base import Arch


class B200(Arch):
    def __init__(self, dev_id=0, require_device=False):
        super().__init__()
        self.reg_cap = 65536
        self.smem_cap = 227 * 1024
        self.num_sm = 148
        self.compute_max_core = 148
        self.max_resident_threads_per_sm = 2048
        self.max_resident_blocks_per_sm = 32
        self.max_registers_per_sm = 64 * 1024
        self.max_registers_per_block = 64 * 1024
        self.max_smem_per_sm = 228 * 1024
        self.max_smem_per_block = 227 * 1024
        self.max_threads_per_block = 1024
        self.warp_size = 32
        self.sm_partition = 4
        self.transaction_size = [32, 128]
        self.l2_cache_size = 126 * 1024          # KiB, like the reference's field
        self.tmem_columns = 512                  # 128 lanes x 512 32-bit columns per SM
        # nominal HBM3e, then the copy bandwidth measured on this pool's B200s
        self.bandwidth = [8000, 6547]
        # fp16 CUDA-core, fp32, fp64, dense fp16 tensor TFLOP/s (nominal)
        self.processing_power = [80.0, 80.0, 40.0, 2250.0]
        self.platform = "CUDA"
        self.compute_capability = "100a"
        self.target = "cuda -arch=sm_100a"
        self.dev_id = dev_id
        try:
            import torch
            if torch.cuda.is_available() and dev_id < torch.cuda.device_count():
                self.device = torch.device(f"cuda:{dev_id}")
                self.num_sm = torch.cuda.get_device_properties(dev_id).multi_processor_count
        except ImportError:
            pass
        if require_device and self.device is None:
            raise RuntimeError(f"Cannot find cuda device {dev_id}.")
