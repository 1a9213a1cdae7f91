"""Wrap any exact top-k into a bucketed approximate one (composition of torch ops).

API of the reference's ``approx_topk/experimental/autobucket.py`` (``bucket``
:10-76, ``bucketed_torch_topk`` :79-95).  This is the slow, generic construction
the reference uses to cross-check its kernel; it is not a kernel and runs on
whatever device the input lives on.  Bucket geometry is the operator's:
interleaved bucket ``c`` = positions ``c, c+b, ...``; contiguous buckets differ
in size by at most one, the longer ones first.
"""

from __future__ import annotations

import torch
from torch import Tensor

from .. import Topk


def _lowest(dtype: torch.dtype):
    return torch.finfo(dtype).min if dtype.is_floating_point else torch.iinfo(dtype).min


def bucket(exact_method: Topk, k_mult: int, k_per_bucket: int, interleaved: bool) -> Topk:
    """Build ``f(xs, k, dim)`` that takes ``k_per_bucket`` items from each of
    ``k * k_mult / k_per_bucket`` buckets with ``exact_method`` and then the
    exact top-``k`` of those."""

    def bucketed(xs: Tensor, k: int, dim: int) -> tuple[Tensor, Tensor]:
        n_candidates = k * k_mult
        if n_candidates % k_per_bucket:
            raise NotImplementedError
        dim %= xs.ndim
        if dim != xs.ndim - 1:
            v, i = bucketed(xs.movedim(dim, -1), k=k, dim=-1)
            return v.movedim(-1, dim), i.movedim(-1, dim)

        n = xs.shape[-1]
        b = n_candidates // k_per_bucket
        depth = -(-n // b)                      # longest bucket
        fill = _lowest(xs.dtype)
        # Position table: entry (c, d) is the row position of the d-th element
        # of bucket c, or n (out of range) where the bucket is shorter.
        c = torch.arange(b, device=xs.device).unsqueeze(1)
        d = torch.arange(depth, device=xs.device).unsqueeze(0)
        if interleaved:
            pos = c + d * b
            pos = torch.where(pos < n, pos, n)
        else:
            base, extra = divmod(n, b)
            sizes = base + (c < extra).long()
            starts = c * base + torch.clamp(c, max=extra)
            pos = torch.where(d < sizes, starts + d, n)
        padded = torch.cat([xs, xs.new_full((*xs.shape[:-1], 1), fill)], dim=-1)
        grid = padded[..., pos]                 # (..., b, depth)
        cand_v, cand_d = exact_method(grid, k=k_per_bucket, dim=-1)
        cand_i = pos.expand(*xs.shape[:-1], b, depth).gather(-1, cand_d)
        cand_v, cand_i = cand_v.flatten(-2), cand_i.flatten(-2)
        val, where = torch.topk(cand_v, k=k, dim=-1, sorted=False)
        return val, cand_i.gather(-1, where)

    return bucketed


def bucketed_torch_topk(
    xs: Tensor,
    k: int,
    dim: int,
    k_mult: int,
    k_per_bucket: int,
    interleaved: bool,
) -> tuple[Tensor, Tensor]:
    """``bucket`` applied to ``torch.topk(sorted=False)``."""

    def exact(xs: Tensor, k: int, dim: int) -> tuple[Tensor, Tensor]:
        return torch.topk(xs, k, dim, sorted=False)

    return bucket(exact, k_mult=k_mult, k_per_bucket=k_per_bucket, interleaved=interleaved)(xs, k, dim)
