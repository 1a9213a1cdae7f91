"""Multi-GPU forms of the operator (one process per GPU, ``torch.distributed``).

The reference is single-GPU.  Two partitionings follow from the structure of
the algorithm:

* **Rows** are independent, so a batch is sharded row-wise and every rank runs
  the plain operator on its rows.  No collective is involved
  (:func:`row_shard`, :func:`topk_row_sharded`).

* **One very long row** with interleaved buckets is a ``stripes x b`` matrix;
  rank ``g`` of ``G`` owns the contiguous *bucket group* (columns)
  ``[g*b/G, (g+1)*b/G)`` as a dense ``stripes x b/G`` slab in its own memory.
  Stage 1 is independent per bucket, so each rank produces exactly the slice
  ``[g*k0/G, (g+1)*k0/G)`` of the single-GPU candidate buffer (slot =
  ``bucket*j + q``).  One all-gather of the (value, index) candidates over
  NVLink reassembles that buffer on every rank, and the exact select over it
  gives the same answer as one GPU would (:func:`topk_long_row`).

The candidates land in each GPU's own memory before the select reads them; no
kernel touches a peer's memory.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist
from torch import Tensor

from . import _native


def row_shard(rows: int, rank: int, world: int) -> tuple[int, int]:
    """Half-open row range of ``rank`` when ``rows`` rows are split as evenly as
    possible over ``world`` ranks (the first ``rows % world`` ranks get one more)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def topk_row_sharded(xs_local: Tensor, k: int, j: int = 1, k_mult: int = 1,
                     interleaved: bool = True) -> tuple[Tensor, Tensor]:
    """The operator on this rank's rows.  Exists for symmetry with
    :func:`topk_long_row`; it is the plain operator because rows never interact."""
    from .priority_queue import topk

    return topk(xs_local, k, -1, j=j, k_mult=k_mult, interleaved=interleaved)


def bucket_group(total_buckets: int, rank: int, world: int) -> tuple[int, int]:
    """Columns ``[start, stop)`` of the ``stripes x total_buckets`` view owned by ``rank``.
    Equal groups are required so that the gathered candidate buffer is dense."""
    if total_buckets % world:
        raise ValueError(f"the number of buckets ({total_buckets}) must be a multiple of the world size ({world})")
    cols = total_buckets // world
    return rank * cols, (rank + 1) * cols


def slab_of_row(row: Tensor, total_buckets: int, rank: int, world: int) -> Tensor:
    """Cut this rank's dense ``stripes x cols`` slab out of a full row (used by
    tests and single-node drivers that start from the whole row)."""
    n = row.numel()
    if n % total_buckets:
        raise ValueError("the row length must be a multiple of the number of buckets")
    start, stop = bucket_group(total_buckets, rank, world)
    return row.view(n // total_buckets, total_buckets)[:, start:stop].contiguous()


def _native_stage1_slab(slab: Tensor, total_buckets: int, col_offset: int, j: int) -> tuple[Tensor, Tensor]:
    _native.require_cuda(slab)
    _native.require_device(slab.device)
    # the kernel reads a dense stripes x cols array: a strided view (a column
    # range cut out of the full row) is copied, never read through its base pointer
    slab = slab.contiguous()
    stripes, cols = slab.shape
    vals = torch.empty(cols * j, device=slab.device, dtype=slab.dtype)
    idx = torch.empty(cols * j, device=slab.device, dtype=torch.int64)
    lib = _native.lib()
    code = _native.dtype_code(slab.dtype)
    with torch.cuda.device(slab.device):
        ws_bytes = lib.atk_stage1_slab_workspace_bytes(code, stripes, cols, j)
        ws = torch.empty(ws_bytes, device=slab.device, dtype=torch.uint8) if ws_bytes else None
        status = lib.atk_stage1_slab(
            slab.data_ptr(), code, stripes, cols, total_buckets, col_offset, j,
            vals.data_ptr(), idx.data_ptr(), ws.data_ptr() if ws is not None else None, ws_bytes,
            _native.current_stream_ptr(slab.device))
    _native.check(status)
    return vals, idx


def _native_select(cand_vals: Tensor, cand_idx: Tensor, k: int) -> tuple[Tensor, Tensor]:
    _native.require_cuda(cand_vals)
    k0 = cand_vals.numel()
    code = _native.dtype_code(cand_vals.dtype)
    lib = _native.lib()
    vals = torch.empty(k, device=cand_vals.device, dtype=cand_vals.dtype)
    idx = torch.empty(k, device=cand_vals.device, dtype=torch.int64)
    with torch.cuda.device(cand_vals.device):
        ws_bytes = lib.atk_select_workspace_bytes(code, 1, k0, k)
        ws = torch.empty(ws_bytes, device=cand_vals.device, dtype=torch.uint8) if ws_bytes else None
        status = lib.atk_select(cand_vals.data_ptr(), cand_idx.data_ptr(), code, 1, k0, k0, k,
                                vals.data_ptr(), idx.data_ptr(), k,
                                ws.data_ptr() if ws is not None else None, ws_bytes,
                                _native.current_stream_ptr(cand_vals.device))
    _native.check(status)
    return vals, idx


def topk_long_row(
    slab: Tensor,
    k: int,
    j: int,
    k_mult: int,
    group: dist.ProcessGroup | None = None,
    stage1: Callable[[Tensor, int, int, int], tuple[Tensor, Tensor]] | None = None,
    select: Callable[[Tensor, Tensor, int], tuple[Tensor, Tensor]] | None = None,
) -> tuple[Tensor, Tensor]:
    """Approximate top-k of one long interleaved row sharded by bucket groups.

    :param slab: this rank's dense ``stripes x cols`` slab (columns
        ``[rank*cols, (rank+1)*cols)`` of the ``stripes x b`` view, ``b = k*k_mult/j``).
    :returns: the ``k`` selected ``(values, indices)``, identical on every rank
        and identical to the single-GPU result; indices are positions in the
        full row.

    ``stage1`` / ``select`` default to the native kernels; they are parameters so
    that the partitioning and the exchange can be exercised on CPU ranks.
    """
    if k_mult < 1:
        raise ValueError(f"k_mult must be >=1, was {k_mult}")
    k0 = k * k_mult
    if k0 % j:
        raise RuntimeError("topk: j must divide k")
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    total_buckets = k0 // j
    start, stop = bucket_group(total_buckets, rank, world)
    if slab.ndim != 2 or slab.shape[1] != stop - start:
        raise ValueError(f"slab must be stripes x {stop - start}, got {tuple(slab.shape)}")
    stage1 = stage1 or _native_stage1_slab
    select = select or _native_select

    local_vals, local_idx = stage1(slab, total_buckets, start, j)
    if world > 1:
        cand_vals = torch.empty(k0, device=slab.device, dtype=slab.dtype)
        cand_idx = torch.empty(k0, device=slab.device, dtype=torch.int64)
        # rank g's candidates are slots [g*k0/G, (g+1)*k0/G): a plain all-gather
        dist.all_gather_into_tensor(cand_vals, local_vals, group=group)
        dist.all_gather_into_tensor(cand_idx, local_idx, group=group)
    else:
        cand_vals, cand_idx = local_vals, local_idx
    if k0 == k:
        return cand_vals, cand_idx
    return select(cand_vals, cand_idx, k)
