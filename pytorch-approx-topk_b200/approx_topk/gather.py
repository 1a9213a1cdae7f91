"""Gather of the records the operator selected (the step after the operator).

Not part of the reference package: its users follow ``approx_topk.topk`` with
``torch.gather`` / ``index_select`` to fetch, for instance, the keys and values
of the selected positions of an attention head.  :func:`gather_records` does
that step with the library's own kernel on the indices the operator returns.
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import _native


def gather_records(src: Tensor, indices: Tensor) -> Tensor:
    """``out[..., q, :] = src[..., indices[..., q], :]``.

    :param src: ``[..., n, d]`` CUDA tensor, the last axis contiguous; the batch
        axes must match those of ``indices`` and collapse onto one stride (a
        contiguous tensor always does).
    :param indices: ``[..., k]`` int64 positions along axis ``-2`` of ``src``
        (what ``approx_topk.topk`` returns for ``dim=-1`` over the ``n`` scores).
    :returns: ``[..., k, d]`` tensor of ``src``'s dtype.  A position outside
        ``[0, n)`` gives a zero record.
    """
    _native.require_cuda(src)
    if indices.dtype != torch.int64 or indices.device != src.device:
        raise ValueError("indices must be an int64 tensor on the device of src")
    if src.ndim < 2 or indices.ndim != src.ndim - 1 or indices.shape[:-1] != src.shape[:-2]:
        raise ValueError(f"shapes do not match: src {tuple(src.shape)}, indices {tuple(indices.shape)}")
    n, d = src.shape[-2], src.shape[-1]
    k = indices.shape[-1]
    batch = list(src.shape[:-2])
    out = torch.empty(batch + [k, d], device=src.device, dtype=src.dtype)
    if out.numel() == 0:
        return out
    src3 = src.reshape(-1, n, d)
    if src3.stride(2) != 1 or src3.stride(1) != d:
        src3 = src3.contiguous()
    idx2 = indices.reshape(-1, k)
    if idx2.stride(1) != 1:
        idx2 = idx2.contiguous()
    rows = src3.shape[0]
    _native.require_device(src.device)
    es = src.element_size()
    with torch.cuda.device(src.device):
        status = _native.lib().atk_gather_records(
            src3.data_ptr(), rows, n, d * es, src3.stride(0) * es if rows > 1 else n * d * es,
            idx2.data_ptr(), k, idx2.stride(0) if rows > 1 else k, out.data_ptr(),
            _native.current_stream_ptr(src.device))
    _native.check(status)
    return out
