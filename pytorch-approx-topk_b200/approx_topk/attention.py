"""Key selection for single-query attention without materialising the scores.

``score_topk(q, keys, k, j, k_mult, scale)`` is
``approx_topk.topk((q @ keys.transpose(-1, -2) * scale).to(q.dtype), k, -1, j, k_mult)``
with the scores produced inside the kernel: the step *before* the operator in the
attention-score use case of the reference's paper (its users run the matrix
product first and hand the scores to ``approx_topk.topk``).  The products are
accumulated in float32 and the scaled sum is rounded once to the element type, so
results agree with a torch matrix product up to the rounding of sums that a different
accumulation order moves across a rounding boundary (about one score in 10^4 differs
by one unit in the last place).  ``scores(q, keys, scale)`` writes the same scores to
memory: ``score_topk`` returns exactly ``approx_topk.topk`` of them.
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import _native


def _check(q: Tensor, keys: Tensor) -> tuple[int, int, int, list[int]]:
    if q.dtype != keys.dtype or q.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("score_topk: q and keys must both be float16 or both bfloat16")
    if keys.ndim != q.ndim + 1 or keys.shape[:-2] != q.shape[:-1] or keys.shape[-1] != q.shape[-1]:
        raise ValueError(f"score_topk: keys must be [..., n, d] for q [..., d]; got {tuple(keys.shape)} and {tuple(q.shape)}")
    d = q.shape[-1]
    if d not in (64, 128):
        raise NotImplementedError("score_topk: d must be 64 or 128")
    _native.require_cuda(q)
    _native.require_cuda(keys)
    _native.require_device(q.device)
    lead = list(q.shape[:-1])
    rows = 1
    for s in lead:
        rows *= s
    return rows, keys.shape[-2], d, lead


def scores(q: Tensor, keys: Tensor, scale: float | None = None) -> Tensor:
    """The scores ``(q . keys^T) * scale`` rounded to the input dtype, ``[..., n]``, computed
    with the arithmetic of :func:`score_topk` (bit for bit)."""
    rows, n, d, lead = _check(q, keys)
    if scale is None:
        scale = d ** -0.5
    out = torch.empty(lead + [n], device=q.device, dtype=q.dtype)
    if rows == 0 or n == 0:
        return out
    q2 = q.reshape(rows, d).contiguous()
    k3 = keys.reshape(rows, n, d).contiguous()
    with torch.cuda.device(q.device):
        status = _native.lib().atk_scores(q2.data_ptr(), k3.data_ptr(), _native.dtype_code(q.dtype), rows, n, d, d, n * d,
                                          float(scale), out.data_ptr(), n, _native.current_stream_ptr(q.device))
    _native.check(status)
    return out


def score_topk(q: Tensor, keys: Tensor, k: int, j: int = 1, k_mult: int = 1,
               scale: float | None = None) -> tuple[Tensor, Tensor]:
    """Approximate top-k keys by score for one query per row.

    :param q: ``[..., d]`` float16 / bfloat16 CUDA tensor, ``d`` = 64 or 128.
    :param keys: ``[..., n, d]`` of the same dtype and leading shape, contiguous.
    :param scale: multiplier of the dot products, default ``d ** -0.5``.
    :returns: ``(values [..., k], indices [..., k] int64)``; ``values`` are the scores
        rounded to the input dtype, ``indices`` positions along ``n``.
    """
    if k_mult < 1:
        raise ValueError(f"k_mult must be >=1, was {k_mult}")
    rows, n, d, lead = _check(q, keys)
    q2 = q.reshape(rows, d).contiguous()
    k3 = keys.reshape(rows, n, d).contiguous()
    if scale is None:
        scale = d ** -0.5
    values = torch.empty(lead + [k], device=q.device, dtype=q.dtype)
    indices = torch.empty(lead + [k], device=q.device, dtype=torch.int64)
    if rows == 0 or k == 0:
        return values, indices
    lib = _native.lib()
    code = _native.dtype_code(q.dtype)
    with torch.cuda.device(q.device):
        ws_bytes = lib.atk_score_topk_workspace_bytes(code, rows, n, k, j, k_mult)
        ws = torch.empty(ws_bytes, device=q.device, dtype=torch.uint8) if ws_bytes else None
        status = lib.atk_score_topk(q2.data_ptr(), k3.data_ptr(), code, rows, n, d, d, n * d, float(scale), k, j, k_mult,
                                    values.data_ptr(), indices.data_ptr(), k,
                                    ws.data_ptr() if ws is not None else None, ws_bytes,
                                    _native.current_stream_ptr(q.device))
    _native.check(status)
    return values, indices
