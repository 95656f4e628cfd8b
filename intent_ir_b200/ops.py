"""Device-resident entry points: torch CUDA tensors in, torch CUDA tensors out, no host
copies, no synchronisation.  Each function checks its tensors the way the reference's
generated launch wrapper does (``is_cuda`` / ``is_contiguous`` / dtype,
frontends/cuda/runtime.py:641-669), enqueues the kernel on torch's current stream
(:723, :731) through the C ABI and returns.  PyTorch only allocates the buffers.
"""

from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Sequence, Tuple

import torch

from . import _lib
from .errors import B200LoweringError, B200RuntimeError

_TORCH_CODE = {
    torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.int32: _lib.I32,
    torch.int64: _lib.I64, torch.bool: _lib.BOOL, torch.uint8: _lib.U8, torch.int8: _lib.I8, torch.int16: _lib.I16,
    torch.float64: _lib.F64,
}
TORCH_OF_DTYPE = {
    "f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16, "i32": torch.int32, "i64": torch.int64,
    "bool": torch.bool, "i1": torch.bool, "u8": torch.uint8, "i8": torch.int8, "i16": torch.int16, "f64": torch.float64,
}


def _check(rc: int, what: str) -> None:
    if rc == _lib.OK:
        return
    msg = f"{what}: {_lib.last_error()} (status {rc})"
    if rc == _lib.ERR_UNSUPPORTED:
        raise B200LoweringError(msg)
    raise B200RuntimeError(msg)


def _dev(t: torch.Tensor, name: str) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise B200RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise B200RuntimeError(f"{name} must be contiguous")
    return t


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else (t.data_ptr() or None)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def code_of(t: torch.Tensor) -> int:
    try:
        return _TORCH_CODE[t.dtype]
    except KeyError:
        raise B200LoweringError(f"unsupported tensor dtype {t.dtype}") from None


# ---- device status word for the bounded waits of the tensor-core GEMM -----------------------
_status: Dict[int, torch.Tensor] = {}


def status_word() -> torch.Tensor:
    dev = torch.cuda.current_device()
    if dev not in _status:
        _status[dev] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{dev}")
    return _status[dev]


def check_device_status() -> None:
    """Synchronise the current stream and raise if a bounded device-side wait expired."""
    dev = torch.cuda.current_device()
    if dev not in _status:
        return
    rc = _lib.load().ib200_check_status(_status[dev].data_ptr(), _stream())
    if rc != _lib.OK:
        msg = _lib.last_error()
        _status[dev].zero_()
        raise B200RuntimeError(msg)


# ---- ops ------------------------------------------------------------------------------------

def normalise_axes(dims: Sequence[int], rank: int) -> Tuple[int, ...]:
    axes = sorted({d + rank if d < 0 else d for d in dims})
    if any(a < 0 or a >= rank for a in axes):
        raise B200LoweringError(f"reduce axes {list(dims)} out of range for rank {rank}")
    return tuple(axes)


def reduce(x: torch.Tensor, kind: str, dims: Sequence[int], keepdims: bool = False, scale: float = 1.0,
           out_dtype: Optional[torch.dtype] = None, split: bool = True) -> torch.Tensor:
    """``reduce_sum`` / ``reduce_max`` / ``reduce_any`` over a contiguous run of axes.  With
    ``split`` (default) shapes with too few results to fill the GPU get scratch memory and are
    split along the reduced axis; the result does not vary from run to run either way."""
    _dev(x, "x")
    axes = normalise_axes(dims, x.dim())
    if not axes:
        raise B200LoweringError("reduce needs at least one axis")
    if axes != tuple(range(axes[0], axes[-1] + 1)):
        raise B200LoweringError(f"reduce axes {axes} are not adjacent")
    shape = list(x.shape)
    outer = int(torch.Size(shape[: axes[0]]).numel())
    red = int(torch.Size(shape[axes[0]: axes[-1] + 1]).numel())
    inner = int(torch.Size(shape[axes[-1] + 1:]).numel())
    kinds = {"sum": _lib.REDUCE_SUM, "max": _lib.REDUCE_MAX, "any": _lib.REDUCE_ANY}
    if out_dtype is None:
        out_dtype = torch.bool if kind == "any" else x.dtype
    out_shape = [1 if i in axes else d for i, d in enumerate(shape)] if keepdims else [d for i, d in enumerate(shape) if i not in axes]
    out = torch.empty(out_shape, dtype=out_dtype, device=x.device)
    lib = _lib.load()
    need = int(lib.ib200_reduce_scratch_bytes(outer, red, inner)) if split else 0
    if need:
        scratch = torch.empty(need, dtype=torch.uint8, device=x.device)  # freed stream-ordered by the caching allocator
        rc = lib.ib200_reduce_ws(_ptr(x), _ptr(out), code_of(x), code_of(out), kinds[kind], outer, red, inner, float(scale),
                                 _ptr(scratch), need, _stream())
    else:
        rc = lib.ib200_reduce(_ptr(x), _ptr(out), code_of(x), code_of(out), kinds[kind], outer, red, inner, float(scale), _stream())
    _check(rc, f"reduce_{kind}")
    return out


def softmax(x: torch.Tensor, out: Optional[torch.Tensor] = None, row_max: Optional[torch.Tensor] = None,
            row_sum: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Softmax over the last axis.  ``out_dtype`` (or the dtype of ``out``) may be float32 for
    bf16 / f16 inputs."""
    _dev(x, "x")
    cols = x.shape[-1] if x.dim() else 1
    rows = x.numel() // cols if cols else 0
    if out is None:
        out = torch.empty_like(x, dtype=out_dtype or x.dtype)
    _dev(out, "out")
    for t, n in ((row_max, "row_max"), (row_sum, "row_sum")):
        if t is not None and (_dev(t, n).dtype != torch.float32 or t.numel() != rows):
            raise B200RuntimeError(f"{n} must be f32 with one element per row")
    rc = _lib.load().ib200_softmax_io(_ptr(x), _ptr(out), _ptr(row_max), _ptr(row_sum), code_of(x), code_of(out), rows, cols, _stream())
    _check(rc, "softmax")
    return out


def softmax_masked(x: torch.Tensor, mask: torch.Tensor, fill: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``softmax(where(mask, x, fill))`` over the last axis of an f32 tensor in one kernel.  ``mask``
    (bool / uint8) has the shape of ``x`` or of its last axis (one vector shared by all rows)."""
    _dev(x, "x")
    _dev(mask, "mask")
    if x.dtype != torch.float32 or mask.dtype not in (torch.bool, torch.uint8):
        raise B200RuntimeError("softmax_masked: x must be float32 and mask bool or uint8")
    cols = x.shape[-1] if x.dim() else 1
    rows = x.numel() // cols if cols else 0
    if tuple(mask.shape) == tuple(x.shape):
        stride = cols
    elif mask.numel() == cols:
        stride = 0
    else:
        raise B200RuntimeError(f"softmax_masked: mask shape {tuple(mask.shape)} matches neither x {tuple(x.shape)} nor its last axis")
    if out is None:
        out = torch.empty_like(x)
    _dev(out, "out")
    rc = _lib.load().ib200_softmax_masked(_ptr(x), _ptr(mask), stride, float(fill), _ptr(out), None, None, rows, cols, _stream())
    _check(rc, "softmax_masked")
    return out


def norm_rows(x, w, b, rows: int, cols: int, affine_inner: int, affine_period: int, eps: float, want_stats: bool = True):
    _dev(x, "x")
    y = torch.empty_like(x)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device) if want_stats else None
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device) if want_stats else None
    aff = w if w is not None else b
    if w is not None and b is not None and w.dtype != b.dtype:
        raise B200LoweringError("norm: weight and bias must share a dtype")
    for t, n in ((w, "w"), (b, "b")):
        if t is not None:
            _dev(t, n)
    rc = _lib.load().ib200_norm_rows(
        _ptr(x), _ptr(w), _ptr(b), _ptr(y), _ptr(mean), _ptr(rstd), code_of(x), code_of(aff) if aff is not None else code_of(x),
        rows, cols, affine_inner, affine_period, float(eps), _stream())
    _check(rc, "norm_rows")
    return y, mean, rstd


def layernorm(x: torch.Tensor, w: Optional[torch.Tensor], b: Optional[torch.Tensor], eps: float = 1e-5):
    """y, mean[rows], rstd[rows] over the last axis of x."""
    cols = x.shape[-1]
    return norm_rows(x, w, b, x.numel() // max(cols, 1), cols, 1, cols, eps)


def groupnorm(x: torch.Tensor, w: Optional[torch.Tensor], b: Optional[torch.Tensor], groups: int, eps: float = 1e-5):
    """x is [N, C, *spatial]; returns y, mean[N, G], rstd[N, G]."""
    n, c = x.shape[0], x.shape[1]
    hw = x.numel() // max(n * c, 1)
    if groups <= 0 or c % groups:
        raise B200LoweringError(f"groupnorm: C={c} is not a multiple of groups={groups}")
    y, mean, rstd = norm_rows(x, w, b, n * groups, (c // groups) * hw, max(hw, 1), max(c, 1), eps)
    return y, mean.view(n, groups), rstd.view(n, groups)


_gemm_scratch: Dict[int, torch.Tensor] = {}


def gemm_bias_act(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
                  transpose_b: bool = False, out_dtype: Optional[torch.dtype] = None, allow_tf32: bool = False,
                  split_tail: bool = True, cta_pairs: Optional[bool] = None, narrow_tail: bool = False) -> torch.Tensor:
    """act(a @ b + bias) with fp32 accumulation; ``b`` is [K,N], or [N,K] with transpose_b.  bf16 / f16 operands
    (and f32 operands with ``allow_tf32``) whose K and N are multiples of 8 run on the tensor cores.  ``split_tail``
    gives the kernel scratch memory (kept per device, grown on demand) so that a last, mostly empty round of tiles
    is split along K.  ``cta_pairs``: True / False force the two-CTA (cta_group::2) or the one-CTA kernel; None lets the
    library choose (pairs for large products).  ``narrow_tail`` runs the pair kernel's last-round tiles as two half-width units each when they fill at most half of the pairs."""
    _dev(a, "a"), _dev(b, "b")
    if a.dim() != 2 or b.dim() != 2 or a.dtype != b.dtype:
        raise B200LoweringError("gemm: a and b must be rank-2 tensors of one dtype")
    m, k = a.shape
    n = b.shape[0] if transpose_b else b.shape[1]
    if (b.shape[1] if transpose_b else b.shape[0]) != k:
        raise B200LoweringError(f"gemm: inner extents differ: {tuple(a.shape)} x {tuple(b.shape)}")
    out_dtype = out_dtype or a.dtype
    c = torch.empty((m, n), dtype=out_dtype, device=a.device)
    if bias is not None:
        _dev(bias, "bias")
        if bias.dtype != out_dtype or bias.numel() != n:
            raise B200LoweringError("gemm: bias must have the output dtype and N elements")
    lib = _lib.load()
    flags = (_lib.GEMM_ALLOW_TF32 if allow_tf32 else 0) | (_lib.GEMM_CTA_PAIRS if cta_pairs else _lib.GEMM_ONE_CTA if cta_pairs is False else 0)
    flags |= _lib.GEMM_NARROW_TAIL if narrow_tail else 0
    need = lib.ib200_gemm_scratch_bytes(code_of(a), code_of(c), m, n, k, int(transpose_b), flags) if split_tail else 0
    scratch = None
    if need:
        dev = a.device.index if a.device.index is not None else torch.cuda.current_device()
        scratch = _gemm_scratch.get(dev)
        if scratch is None or scratch.numel() < need + 256:
            scratch = _gemm_scratch[dev] = torch.empty(need + 256, dtype=torch.uint8, device=a.device)
    rc = lib.ib200_gemm_bias_act_ws(
        _ptr(a), _ptr(b), _ptr(bias), _ptr(c), code_of(a), code_of(c), m, n, k, int(transpose_b),
        {"none": _lib.ACT_NONE, "relu": _lib.ACT_RELU}[act], flags, ((scratch.data_ptr() + 255) & ~255) if need else None, need,
        status_word().data_ptr(), _stream())
    _check(rc, "gemm_bias_act")
    return c


def transpose2d(x: torch.Tensor) -> torch.Tensor:
    _dev(x, "x")
    if x.dim() != 2:
        raise B200LoweringError("transpose2d needs a rank-2 tensor")
    out = torch.empty((x.shape[1], x.shape[0]), dtype=x.dtype, device=x.device)
    rc = _lib.load().ib200_transpose2d(_ptr(x), _ptr(out), x.element_size(), x.shape[0], x.shape[1], _stream())
    _check(rc, "transpose2d")
    return out
