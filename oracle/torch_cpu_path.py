"""The reference's CPU-runnable path, restated with torch CPU ops (test / baseline
infrastructure only; the product never imports this).

The reference has no CPU kernel of its own: on CPU tensors its path is the
composition of ATen ops in
  approx_topk/experimental/autobucket.py:10-95   (any j, k_mult: pad, view as
      buckets, torch.topk per bucket, index fix-up, final torch.topk + gather)
  approx_topk/experimental/bucketed_argmax.py:18-42  (k_b = 1: pad, view, max)
This module follows those steps one for one so that timing it on the host's
cores gives the "reference CPU path" baseline that is reported beside the GPU
numbers; ATen parallelises the ops over the threads torch is given.
"""

from __future__ import annotations

import torch
from torch import Tensor
from torch.nn.functional import pad


def _lowest(dtype: torch.dtype):
    return torch.finfo(dtype).min if dtype.is_floating_point else torch.iinfo(dtype).min


def bucketed_topk_cpu(xs: Tensor, k: int, j: int, k_mult: int, interleaved: bool = True) -> tuple[Tensor, Tensor]:
    """autobucket.bucket(torch.topk(sorted=False), k_mult, j, interleaved)(xs, k, -1)."""
    k0 = k * k_mult
    if k0 % j:
        raise NotImplementedError
    n = xs.size(-1)
    b = k0 // j
    n_pad = -n % b
    if interleaved:
        # autobucket.py:40-50 — pad the tail, view (stripes, b), make buckets rows
        xp = pad(xs, (0, n_pad), value=_lowest(xs.dtype))
        per_bucket = xp.unflatten(-1, (-1, b)).transpose(-1, -2)
        v0, i0 = torch.topk(per_bucket, j, dim=-1, sorted=False)
        i0 = i0 * b + torch.arange(b, dtype=torch.int64).unsqueeze(-1)
    else:
        # autobucket.py:52-69 — balanced segments, the first n % b one longer
        depth = (n + n_pad) // b
        buf = torch.full((*xs.shape[:-1], b, depth), _lowest(xs.dtype), dtype=xs.dtype)
        mask = torch.ones((b, depth), dtype=torch.bool)
        mask[(n % b or b):, -1] = False
        buf[..., mask] = xs
        v0, i0 = torch.topk(buf, j, dim=-1, sorted=False)
        starts = torch.cumsum(mask.sum(-1), 0) - mask.sum(-1)
        i0 = i0 + starts.unsqueeze(-1)
    # autobucket.py:72-74 — always a final exact top-k over the candidates
    v, where = torch.topk(v0.flatten(-2), k, dim=-1, sorted=False)
    return v, i0.flatten(-2).gather(-1, where)


def bucketed_argmax_cpu(xs: Tensor, k: int, interleaved: bool = True) -> tuple[Tensor, Tensor]:
    """bucketed_argmax.topk_torch(xs, k, -1, interleaved) (bucketed_argmax.py:18-42)."""
    n = xs.size(-1)
    xp = pad(xs, (0, -n % k), value=_lowest(xs.dtype))
    ks = torch.arange(k, dtype=torch.int64)
    if interleaved:
        m = xp.unflatten(-1, (-1, k)).max(dim=-2)
        return m.values, m.indices * k + ks
    m = xp.unflatten(-1, (k, -1)).max(dim=-1)
    return m.values, m.indices + (xp.size(-1) // k) * ks
