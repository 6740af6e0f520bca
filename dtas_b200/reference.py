"""Input generators for profiling and parity runs.

`get_ref_tensor` mirrors the reference helper of the same name
(python/dtas/reference.py:8-16: uniform(0,1) floats, randint(0,100) integers) on torch.
`seeded_normal` produces the seeded N(mean, scale) tensors the measured configurations use;
it always draws fp32 on the CPU generator and casts afterwards, so the same call yields the
same bits on every machine, for the device run and for the CPU checker alike.
"""
import torch

_TORCH_DTYPE = {"float16": torch.float16, "float32": torch.float32, "int8": torch.int8}


def torch_dtype(name):
    return _TORCH_DTYPE[name] if isinstance(name, str) else name


def get_ref_tensor(shape, device, dtype):
    dtype = torch_dtype(dtype)
    if dtype.is_floating_point:
        return torch.rand(tuple(shape), dtype=torch.float32).to(dtype).to(device)
    return torch.randint(0, 100, tuple(shape), dtype=dtype).to(device)


def seeded_normal(shape, seed, dtype="float16", scale=1.0, mean=0.0):
    """CPU tensor ~ N(mean, scale^2), drawn as fp32 from `seed`, then cast to `dtype`."""
    g = torch.Generator("cpu").manual_seed(int(seed))
    t = torch.randn(tuple(shape), generator=g, dtype=torch.float32)
    if scale != 1.0:
        t = t * scale
    if mean != 0.0:
        t = t + mean
    dtype = torch_dtype(dtype)
    if dtype == torch.int8:
        return (t * 40).round().clamp(-128, 127).to(torch.int8)
    return t.to(dtype)


def config_seed(config_index, tensor_index):
    """Seed of tensor `tensor_index` of measured configuration `config_index` (0-based)."""
    return 1000 * int(config_index) + int(tensor_index)
