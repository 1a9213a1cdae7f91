"""Narrow output formats of the operator (opt-in; the default API is unchanged).

The reference always returns int64 indices (``approx_topk/priority_queue.py:65-67``).
A consumer that only needs 32-bit positions (every row shorter than 2^31) can ask
the same kernels to store them as int32, or as packed 8-byte records
``{value bits, int32 position}`` that are read back with one load per pair: on the
headline workload the int64 indices are two thirds of all bytes written.  The
selection itself, and the order of the pairs inside a row, are exactly those of
:func:`approx_topk.topk`.
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import _native


def topk_narrow(xs: Tensor, k: int, dim: int = -1, j: int = 1, k_mult: int = 1,
                records: bool = False) -> tuple[Tensor, Tensor] | Tensor:
    """``approx_topk.topk(xs, k, dim, j, k_mult)`` (interleaved buckets) with 32-bit positions.

    :param records: ``False``: returns ``(values, indices)`` with ``indices`` of dtype
        int32.  ``True``: returns ONE int32 tensor ``[..., k, 2]`` of packed records,
        ``[..., 0]`` holding the bits of the value (zero-extended to 32 bits; for
        float32 ``rec[..., 0].view(torch.float32)`` are the values) and ``[..., 1]``
        the position.  Element types of at most 32 bits.
    :raises RuntimeError: if a row has 2^31 or more elements.
    """
    dim = dim % xs.ndim
    if dim != xs.ndim - 1:
        raise NotImplementedError("the narrow formats are built for the last dimension")
    if k_mult < 1:
        raise ValueError(f"k_mult must be >=1, was {k_mult}")
    _native.require_cuda(xs)
    _native.require_device(xs.device)
    code = _native.dtype_code(xs.dtype)
    x2, rows, n, row_stride = _native.as_rows(xs)
    lead = list(xs.shape[:-1])
    lib = _native.lib()
    with torch.cuda.device(xs.device):
        ws_bytes = lib.atk_topk_workspace_bytes(code, rows, n, k, j, k_mult)
        ws = torch.empty(ws_bytes, device=xs.device, dtype=torch.uint8) if ws_bytes else None
        if records:
            out = torch.empty(lead + [k, 2], device=xs.device, dtype=torch.int32)
            status = lib.atk_topk_ex(x2.data_ptr(), code, rows, n, row_stride, k, j, k_mult, 1, -1,
                                     _native.ATK_OUT_REC32, out.data_ptr(), None, k,
                                     ws.data_ptr() if ws is not None else None, ws_bytes,
                                     _native.current_stream_ptr(xs.device))
            _native.check(status)
            return out
        values = torch.empty(lead + [k], device=xs.device, dtype=xs.dtype)
        indices = torch.empty(lead + [k], device=xs.device, dtype=torch.int32)
        status = lib.atk_topk_ex(x2.data_ptr(), code, rows, n, row_stride, k, j, k_mult, 1, -1,
                                 _native.ATK_OUT_I32, values.data_ptr(), indices.data_ptr(), k,
                                 ws.data_ptr() if ws is not None else None, ws_bytes,
                                 _native.current_stream_ptr(xs.device))
    _native.check(status)
    return values, indices
