"""Torch-tensor front end of the C ABI: one function per operator.

Calling convention follows the reference's packed functions: inputs first, the
pre-allocated output last (experiment/dtas_tuned/elementwise/cast/profile_cast.py:15-18);
the symbolic dim is read from the tensor shape, never passed
(experiment/dtas_tuned/elementwise/cast/top10_256/host.cc:52-53).  Tensors may be
`[m, H]` or the reference's `[1, m, H]`.  Every function launches on the current torch
stream of the tensor's device and returns the output tensor.
"""
import torch

from . import _abi

_L = None


def _lib():
    global _L
    if _L is None:
        _L = _abi.lib()
    return _L

_DTYPE_CODE = {torch.float16: _abi.F16, torch.float32: _abi.F32, torch.int8: _abi.I8}


def _chk(status):
    if status:
        _abi.check(status)


def _code(t):
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise _abi.DtasError(_abi.EUNSUPPORTED, f"dtype {t.dtype} has no kernel") from None


def _rows_cols(t, name):
    """[m, H] or [1, m, H] -> (m, H)."""
    if t.dim() == 3 and t.shape[0] == 1:
        return int(t.shape[1]), int(t.shape[2])
    if t.dim() == 2:
        return int(t.shape[0]), int(t.shape[1])
    raise _abi.DtasError(_abi.EINVAL, f"{name}: expected [m, H] or [1, m, H], got {tuple(t.shape)}")


try:   # raw handle of the current stream without building a torch.cuda.Stream object
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:   # older / stripped builds
    def _raw_stream(index):
        return torch.cuda.current_stream(index).cuda_stream


def _check(name, *tensors):
    """Device index and current raw stream; rejects CPU, mixed-device and strided tensors."""
    first = tensors[0]
    if not first.is_cuda:
        raise _abi.DtasError(_abi.EINVAL, f"{name}: tensors must live on a CUDA device, got {first.device}")
    dev = first.device
    for t in tensors:
        if not t.is_contiguous():
            raise _abi.DtasError(_abi.EINVAL, f"{name}: tensors must be contiguous")
        if t.device != dev:
            raise _abi.DtasError(_abi.EINVAL, f"{name}: tensors on different devices")
    index = dev.index
    return index, _raw_stream(index)


def _same_shape(name, a, b):
    if _rows_cols(a, name) != _rows_cols(b, name):
        raise _abi.DtasError(_abi.EINVAL, f"{name}: shape mismatch {tuple(a.shape)} vs {tuple(b.shape)}")


def cast(a, out):
    """out = a converted to out.dtype (fp32 -> fp16 round-to-nearest-even, or fp16 -> fp32)."""
    dev, st = _check("cast", a, out)
    _same_shape("cast", a, out)
    m, h = _rows_cols(a, "cast")
    _chk(_lib().dtas_cast(a.data_ptr(), out.data_ptr(), m, h, _code(a), _code(out), dev, st))
    return out


def add(a, b, out):
    """out = a + b, all three of one dtype (fp16, fp32 or int8)."""
    dev, st = _check("add", a, b, out)
    _same_shape("add", a, b)
    _same_shape("add", a, out)
    if not (a.dtype == b.dtype == out.dtype):
        raise _abi.DtasError(_abi.EINVAL, "add: dtypes differ")
    m, h = _rows_cols(a, "add")
    _chk(_lib().dtas_add(a.data_ptr(), b.data_ptr(), out.data_ptr(), m, h, _code(a), dev, st))
    return out


def copy(a, out):
    """out = a."""
    dev, st = _check("copy", a, out)
    _same_shape("copy", a, out)
    if a.dtype != out.dtype:
        raise _abi.DtasError(_abi.EINVAL, "copy: dtypes differ")
    m, h = _rows_cols(a, "copy")
    _chk(_lib().dtas_copy(a.data_ptr(), out.data_ptr(), m, h, _code(a), dev, st))
    return out


def peer_push(src, dsts):
    """Copies the contiguous tensor `src` to every tensor of `dsts`: views, on this device, of the
    same place in the other ranks' gather buffers (peer memory).  One launch, plain stores over
    NVLink, no cross-rank waiting: run a barrier across ranks before a gathered buffer is read."""
    import ctypes
    dev, st = _check("peer_push", src, *dsts)
    for d in dsts:
        if d.dtype != src.dtype or d.numel() != src.numel():
            raise _abi.DtasError(_abi.EINVAL, "peer_push: destination of another size or dtype")
    ptrs = (ctypes.c_void_p * len(dsts))(*[d.data_ptr() for d in dsts])
    _chk(_lib().dtas_peer_push(src.data_ptr(), ptrs, len(dsts), src.numel() * src.element_size(), dev, st))


def rms_norm(x, weight, out, eps=1e-6):
    """out = x * rsqrt(mean(x^2, -1) + eps) * weight; fp32 arithmetic, fp16 result."""
    dev, st = _check("rms_norm", x, weight, out)
    _same_shape("rms_norm", x, out)
    m, h = _rows_cols(x, "rms_norm")
    if weight.dtype != torch.float16 or weight.numel() != h or out.dtype != torch.float16:
        raise _abi.DtasError(_abi.EINVAL, "rms_norm: weight must be fp16 [H] and out fp16")
    _chk(_lib().dtas_rms_norm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), m, h,
                                        float(eps), _code(x), dev, st))
    return out


def softmax(x, out):
    """out = softmax(x, dim=-1); fp32 arithmetic, fp16 result."""
    dev, st = _check("softmax", x, out)
    _same_shape("softmax", x, out)
    if out.dtype != torch.float16:
        raise _abi.DtasError(_abi.EINVAL, "softmax: out must be fp16")
    m, h = _rows_cols(x, "softmax")
    _chk(_lib().dtas_softmax(x.data_ptr(), out.data_ptr(), m, h, _code(x), dev, st))
    return out


def layer_norm(x, gamma, beta, out, eps=1e-5):
    """out = (x - mean) * rsqrt(var + eps) * gamma + beta; gamma/beta fp32 [H]; fp16 result."""
    dev, st = _check("layer_norm", x, gamma, beta, out)
    _same_shape("layer_norm", x, out)
    m, h = _rows_cols(x, "layer_norm")
    if gamma.dtype != torch.float32 or beta.dtype != torch.float32 or gamma.numel() != h or beta.numel() != h:
        raise _abi.DtasError(_abi.EINVAL, "layer_norm: gamma and beta must be fp32 [H]")
    if out.dtype != torch.float16:
        raise _abi.DtasError(_abi.EINVAL, "layer_norm: out must be fp16")
    _chk(_lib().dtas_layer_norm(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), out.data_ptr(),
                                          m, h, float(eps), _code(x), dev, st))
    return out


_ACTS = {None: _abi.ACT_NONE, "none": _abi.ACT_NONE, "gelu": _abi.ACT_GELU}


def _tail_args(name, out, n, rows, bias, res1, res2, act):
    """Checks the optional tail operands; -> (act code, out dtype code, ldr, fused?)."""
    if act not in _ACTS:
        raise _abi.DtasError(_abi.EINVAL, f"{name}: unknown activation {act!r} (None or 'gelu')")
    if out.dtype not in (torch.float16, torch.float32):
        raise _abi.DtasError(_abi.EUNSUPPORTED, f"{name}: the output must be fp16 or fp32, got {out.dtype}")
    if res1 is None and res2 is not None:
        raise _abi.DtasError(_abi.EINVAL, f"{name}: res2 without res1")
    if bias is not None and (bias.dtype != torch.float16 or bias.numel() != n or not bias.is_contiguous()):
        raise _abi.DtasError(_abi.EINVAL, f"{name}: bias must be a contiguous fp16 vector of N elements")
    ldr = 0
    for r in (res1, res2):
        if r is None:
            continue
        if r.dtype != torch.float16 or r.numel() != rows * n or r.stride(-1) != 1:
            raise _abi.DtasError(_abi.EINVAL, f"{name}: residuals must be fp16 [m, N] with unit inner stride")
        ld = max(int(r.stride(-2)), n) if r.dim() >= 2 else n
        if ldr and ld != ldr and rows > 1:
            raise _abi.DtasError(_abi.EINVAL, f"{name}: both residuals must have the same row stride")
        ldr = ld
    fused = res1 is not None or _ACTS[act] != _abi.ACT_NONE or out.dtype == torch.float32
    return _ACTS[act], (_abi.F32 if out.dtype == torch.float32 else _abi.F16), ldr, fused


def _ptr(t):
    return t.data_ptr() if t is not None else None


def gemv(x, w, out, bias=None, res1=None, res2=None, act=None):
    """out[1, N] = act(x[1, K] @ w[N, K]^T + bias[N]) + res1 + res2; fp16 operands, fp32 accumulation,
    fp16 or fp32 `out` (the fp16 result widened).  bias, res1, res2 and act are optional."""
    tensors = tuple(t for t in (x, w, out, bias, res1, res2) if t is not None)
    dev, st = _check("gemv", *tensors)
    n, k = int(w.shape[0]), int(w.shape[1])
    if w.dim() != 2 or x.numel() != k or out.numel() != n:
        raise _abi.DtasError(_abi.EINVAL, f"gemv: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if not (x.dtype == w.dtype == torch.float16):
        raise _abi.DtasError(_abi.EUNSUPPORTED, "gemv: only fp16 operands are implemented")
    act_c, out_c, _, fused = _tail_args("gemv", out, n, 1, bias, res1, res2, act)
    if fused:
        _chk(_lib().dtas_gemv_fused(x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(res1), _ptr(res2), out.data_ptr(),
                                    n, k, act_c, out_c, _abi.F16, dev, st))
    else:
        _chk(_lib().dtas_gemv(x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), n, k, _abi.F16, dev, st))
    return out


def gemm_nt(x, w, out, bias=None, res1=None, res2=None, act=None):
    """out[m, N] = act(x[m, K] @ w[N, K]^T + bias[N]) + res1[m, N] + res2[m, N]; fp16 operands, fp32
    accumulation, fp16 or fp32 `out` (the fp16 result widened).  bias, res1, res2 and act ('gelu')
    are optional: the fused forms of the reference's model workloads.

    `out` may be a column slab of a wider row-major buffer (last-dim stride 1, any row
    stride >= N): a column-sharded rank writes its part of the full output in place.
    """
    dev_t = x.device
    if dev_t.type != "cuda":
        raise _abi.DtasError(_abi.EINVAL, f"gemm: tensors must live on a CUDA device, got {dev_t}")
    m, k = _rows_cols(x, "gemm")
    mo, n = _rows_cols(out, "gemm")
    if w.dim() != 2 or int(w.shape[1]) != k or int(w.shape[0]) != n or mo != m:
        raise _abi.DtasError(_abi.EINVAL, f"gemm: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if not (x.dtype == w.dtype == torch.float16):
        raise _abi.DtasError(_abi.EUNSUPPORTED, "gemm: only fp16 operands are implemented")
    if not x.is_contiguous() or not w.is_contiguous():
        raise _abi.DtasError(_abi.EINVAL, "gemm: x and w must be contiguous")
    if out.stride(-1) != 1:
        raise _abi.DtasError(_abi.EINVAL, "gemm: out must have unit stride in its last dim")
    ldy = int(out.stride(-2)) if m > 1 else max(int(out.stride(-2)), n)
    for t in (w, out, bias, res1, res2):
        if t is not None and t.device != dev_t:
            raise _abi.DtasError(_abi.EINVAL, "gemm: tensors on different devices")
    act_c, out_c, ldr, fused = _tail_args("gemm", out, n, m, bias, res1, res2, act)
    dev = dev_t.index if dev_t.index is not None else torch.cuda.current_device()
    st = _raw_stream(dev)
    if fused:
        _chk(_lib().dtas_gemm_nt_fused(x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(res1), _ptr(res2), out.data_ptr(),
                                       m, n, k, ldy, ldr, act_c, out_c, _abi.F16, dev, st))
    else:
        _chk(_lib().dtas_gemm_nt(x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), m, n, k, ldy, _abi.F16,
                                 dev, st))
    return out


def gemm_nt_scatter(x, w, out, peers, bias=None, multicast=0):
    """out[m, N] = x[m, K] @ w[N, K]^T (+ bias), and every stored vector of `out` again into each tensor of
    `peers`: views, on this device, with out's shape and row stride - the place of this rank's column
    slab in the other ranks' gather buffers (peer memory).  One launch; the stores to the peers leave
    from the GEMM's epilogue tile by tile.  Run a barrier across ranks before a gathered buffer is read.
    `multicast`, when not 0, is the address of out's slab in a multicast mapping that covers this GPU's
    buffer and every peer's (PeerGatherBuffer.multicast_address): whole blocks then leave as one
    multimem.st per vector and the NVLink switch stores them into every buffer.
    Raises DtasError(EUNSUPPORTED) below 129 rows (use gemm_nt and peer_push there)."""
    import ctypes
    m, k = _rows_cols(x, "gemm_scatter")
    mo, n = _rows_cols(out, "gemm_scatter")
    if x.device.type != "cuda":
        raise _abi.DtasError(_abi.EINVAL, f"gemm_scatter: tensors must live on a CUDA device, got {x.device}")
    if w.dim() != 2 or int(w.shape[1]) != k or int(w.shape[0]) != n or mo != m:
        raise _abi.DtasError(_abi.EINVAL, f"gemm_scatter: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if not (x.dtype == w.dtype == out.dtype == torch.float16) or not x.is_contiguous() or not w.is_contiguous():
        raise _abi.DtasError(_abi.EUNSUPPORTED, "gemm_scatter: contiguous fp16 operands and an fp16 output")
    if out.stride(-1) != 1:
        raise _abi.DtasError(_abi.EINVAL, "gemm_scatter: out must have unit stride in its last dim")
    ldy = int(out.stride(-2)) if m > 1 else max(int(out.stride(-2)), n)
    for p in peers:
        if p.dtype != out.dtype or tuple(p.shape) != tuple(out.shape) or p.stride() != out.stride():
            raise _abi.DtasError(_abi.EINVAL, "gemm_scatter: every peer view must have out's dtype, shape and strides")
    if bias is not None and (bias.dtype != torch.float16 or bias.numel() != n or not bias.is_contiguous()):
        raise _abi.DtasError(_abi.EINVAL, "gemm_scatter: bias must be a contiguous fp16 vector of N elements")
    dev = x.device.index if x.device.index is not None else torch.cuda.current_device()
    ptrs = (ctypes.c_void_p * len(peers))(*[p.data_ptr() for p in peers])
    _chk(_lib().dtas_gemm_nt_scatter_multicast(x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), ptrs, len(peers),
                                               int(multicast) or None, m, n, k, ldy, _abi.F16, dev, _raw_stream(dev)))
    return out


def poll_status(device=None):
    """Synchronises `device` and raises DtasError(ETIMEOUT) if a bounded device-side wait gave up."""
    if device is None:
        device = torch.cuda.current_device()
    _chk(_lib().dtas_poll_status(int(device)))
