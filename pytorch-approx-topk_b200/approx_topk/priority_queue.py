"""The ``approx_topk::topk`` operator on hand-written sm_100a kernels.

Same name, signature, defaults, checks and return types as the reference
operator (reference approx_topk/priority_queue.py:14-104); the body calls the
C-ABI library instead of a JIT-compiled pybind module, and the second stage is
a native exact-select kernel instead of ``torch.topk`` + ``gather``.
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import _native


@torch.library.custom_op("approx_topk::topk", mutates_args=())
def topk(
    xs: Tensor,
    k: int,
    dim: int,
    j: int = 1,
    k_mult: int = 1,
    interleaved: bool = True,
    multithread_buckets: bool | None = False,
) -> tuple[Tensor, Tensor]:
    """Approximate top-k along ``dim``.

    The row is split into ``b = k_mult * k / j`` buckets (interleaved: bucket
    ``c`` holds positions ``c, c+b, c+2b, ...``; otherwise contiguous segments),
    the top ``j`` of every bucket are kept and, when ``k_mult > 1``, an exact
    top-k over those ``b*j`` candidates gives the result.

    :param j: items kept per bucket, 1..4, must divide ``k * k_mult``.
    :param k_mult: bucket-count multiplier; > 1 raises recall and adds the
        exact second stage.
    :param multithread_buckets: accepted for compatibility with the reference,
        where it picks between two kernels; one kernel family serves every
        shape here, so the value does not change the result.
    :returns: ``(values, indices)`` with ``shape[dim] == k``; values in the
        input dtype, indices int64 positions along ``dim``.  Order along
        ``dim`` is unspecified.
    """
    dim = _normalise_dim(xs, dim)
    if dim != xs.ndim - 1 and j < k:
        # several buckets along a strided axis are not supported (same rule as the reference)
        raise NotImplementedError("This topk only currently works on the last dim")
    if k_mult < 1:
        raise ValueError(f"k_mult must be >=1, was {k_mult}")
    k0 = k * k_mult

    _native.require_cuda(xs)
    code = _native.dtype_code(xs.dtype)
    output_shape = _get_output_shape(xs, k, dim)
    if k == 0 or xs.numel() == 0:
        return (torch.empty(output_shape, device=xs.device, dtype=xs.dtype),
                torch.empty(output_shape, device=xs.device, dtype=torch.int64))
    _native.require_device(xs.device)
    lib = _native.lib()

    last = xs.ndim - 1
    x_last = xs if dim == last else xs.movedim(dim, -1)
    x2, rows, n, row_stride = _native.as_rows(x_last)
    lead_shape = list(x_last.shape[:-1])
    values = torch.empty(lead_shape + [k], device=xs.device, dtype=xs.dtype)
    indices = torch.empty(lead_shape + [k], device=xs.device, dtype=torch.int64)

    with torch.cuda.device(xs.device):
        ws_bytes = lib.atk_topk_workspace_bytes(code, rows, n, k, j, k_mult)
        workspace = torch.empty(ws_bytes, device=xs.device, dtype=torch.uint8) if ws_bytes else None
        mode = -1 if multithread_buckets is None else int(bool(multithread_buckets))
        status = lib.atk_topk(
            x2.data_ptr(), code, rows, n, row_stride, k, j, k_mult, int(interleaved), mode,
            values.data_ptr(), indices.data_ptr(), k,
            workspace.data_ptr() if workspace is not None else None, ws_bytes,
            _native.current_stream_ptr(xs.device),
        )
    _native.check(status)
    if dim != last:
        values = values.movedim(-1, dim).contiguous()
        indices = indices.movedim(-1, dim).contiguous()
    return values, indices


def _fake_topk(
    xs: Tensor,
    k: int,
    dim: int,
    j: int | None = None,
    k_mult: int = 1,
    interleaved: bool = True,
    multithread_buckets: bool | None = False,
) -> tuple[Tensor, Tensor]:
    """Meta implementation: shapes and dtypes only (for torch.compile / opcheck)."""
    shape = _get_output_shape(xs, k, dim)
    return xs.new_empty(shape), xs.new_empty(shape, dtype=torch.int64)


topk.register_fake(_fake_topk)


def _normalise_dim(xs: Tensor, dim: int) -> int:
    return dim + xs.ndim if dim < 0 else dim


def _get_output_shape(xs: Tensor, k: int, dim: int) -> list[int]:
    """The input's shape with ``k`` entries along ``dim``."""
    shape = list(xs.shape)
    shape[dim] = k
    return shape
