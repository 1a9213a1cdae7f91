"""k_b = 1 bucketed arg-max entry points, served by the sm_100a kernels.

Keeps the call signatures of the reference module
(reference approx_topk/experimental/bucketed_argmax.py: ``topk_torch`` :18-42,
``_batch_contiguous`` :45-67, ``topk_triton`` :145-202).  Both ``topk_torch``
and ``topk_triton`` run the same native kernel: there is no Triton and no
composition of torch ops on the data path.  Conventions kept from the
reference: ``k`` buckets; rows behave as if padded to a multiple of ``k`` with
the dtype's lowest value; contiguous buckets are fixed chunks of
``ceil(n / k)``; the first maximum wins a tie; outputs are in bucket order.
"""

from __future__ import annotations

from typing import Any, Literal

import torch
from torch import Tensor

from .. import _native


def _min_value(dtype: torch.dtype) -> Any:
    info = torch.finfo(dtype) if dtype.is_floating_point else torch.iinfo(dtype)
    return info.min


def _batch_contiguous(x: Tensor) -> Tensor:
    """Return ``x`` itself when its last axis has unit stride, rows do not
    overlap and all leading axes collapse onto one uniform row stride (so the
    tensor is ``rows x n`` with a single stride between rows); otherwise return
    a contiguous copy."""
    strides, shape = x.stride(), x.shape
    if strides[-1] != 1:
        return x.contiguous()
    if x.ndim < 2:
        return x
    row_stride = strides[-2]
    if row_stride < shape[-1]:
        return x.contiguous()
    # Leading axis i must step over exactly shape[i+1] steps of axis i+1.
    want = row_stride
    for axis in range(x.ndim - 2, -1, -1):
        if strides[axis] != want:
            return x.contiguous()
        want *= shape[axis]
    return x


def _argmax_cuda(xs: Tensor, k: int, dim: int, interleaved: bool) -> tuple[Tensor, Tensor]:
    _native.require_cuda(xs)
    code = _native.dtype_code(xs.dtype)
    dim = dim % xs.ndim
    last = xs.ndim - 1
    x_last = xs if dim == last else xs.movedim(dim, -1)
    x_last = _batch_contiguous(x_last)
    n = x_last.shape[-1]
    rows = x_last.numel() // n if n else 0
    row_stride = x_last.stride(-2) if x_last.ndim >= 2 and rows > 1 else n
    lead = list(x_last.shape[:-1])
    values = torch.empty(lead + [k], device=xs.device, dtype=xs.dtype)
    indices = torch.empty(lead + [k], device=xs.device, dtype=torch.int64)
    if k > 0 and rows > 0:
        _native.require_device(xs.device)
        lib = _native.lib()
        with torch.cuda.device(xs.device):
            ws_bytes = lib.atk_stage1_workspace_bytes(code, rows, n, k, 1, int(interleaved)) if k <= n else 0
            ws = torch.empty(ws_bytes, device=xs.device, dtype=torch.uint8) if ws_bytes else None
            status = lib.atk_bucketed_argmax(
                x_last.data_ptr(), code, rows, n, row_stride, k, int(interleaved),
                values.data_ptr(), indices.data_ptr(), k,
                ws.data_ptr() if ws is not None else None, ws_bytes,
                _native.current_stream_ptr(xs.device),
            )
        _native.check(status)
    if dim != last:
        return values.movedim(-1, dim), indices.movedim(-1, dim)
    return values, indices


def topk_torch(xs: Tensor, k: int, dim: int, interleaved: bool) -> tuple[Tensor, Tensor]:
    """One maximum per bucket, ``k`` buckets along ``dim`` (bucket order)."""
    return _argmax_cuda(xs, k, dim, interleaved)


def topk_triton(
    xs: Tensor,
    k: int,
    dim: int,
    interleaved: bool,
    block_size: int,
    kernel: Literal["bk", "bkn"],
) -> tuple[Tensor, Tensor]:
    """Same result as :func:`topk_torch`.  ``block_size`` and ``kernel`` selected
    a Triton launch shape in the reference; they are validated and otherwise
    ignored because the launch shape is chosen by the native library."""
    if kernel not in ("bk", "bkn"):
        raise ValueError(f"Unknown kernel {kernel!r}")
    if block_size < 1:
        raise ValueError(f"block_size must be positive, was {block_size}")
    return _argmax_cuda(xs, k, dim, interleaved)
