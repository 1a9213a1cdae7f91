"""Approximate top-k for data that lives in host memory.

``topk_host(xs_cpu, k, j, k_mult)`` is the end-to-end form of the operator for
callers whose rows sit in (ideally pinned) host memory: the native library
streams the rows to the GPU in chunks, runs the kernels on each chunk and
streams the results back, overlapping upload, compute and download.  The
reference has no such entry point (its users write ``xs.cuda()`` /
``.cpu()`` around the op); the result is identical to doing exactly that.
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import _native

_scratch_cache: dict[tuple[int, int], Tensor] = {}


def _scratch(device: torch.device, nbytes: int) -> Tensor:
    """Device staging memory, grown on demand and kept per device."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), 0)
    buf = _scratch_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1), device=device, dtype=torch.uint8)
        _scratch_cache[key] = buf
    return buf


def topk_host(
    xs: Tensor,
    k: int,
    j: int = 1,
    k_mult: int = 1,
    interleaved: bool = True,
    device: torch.device | str | int = "cuda",
    chunk_rows: int = 0,
    out: tuple[Tensor, Tensor] | None = None,
) -> tuple[Tensor, Tensor]:
    """Approximate top-k along the last dim of a host tensor; returns host tensors.

    :param xs: CPU tensor ``[..., n]`` (float32 / float16 / bfloat16), contiguous.
        Pinned memory (``xs.pin_memory()``) is needed for full PCIe speed.
    :param out: optional pre-allocated ``(values, indices)`` CPU tensors to fill.
    :param chunk_rows: rows per pipeline chunk; 0 lets the library choose.
    """
    if xs.is_cuda:
        raise RuntimeError("topk_host expects a CPU tensor; use approx_topk.topk for CUDA tensors")
    if k_mult < 1:
        raise ValueError(f"k_mult must be >=1, was {k_mult}")
    code = _native.dtype_code(xs.dtype)
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("topk_host needs a CUDA device to run on")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    _native.require_device(device)
    xs = xs.contiguous()
    n = xs.shape[-1]
    rows = xs.numel() // n if n else 0
    lead = list(xs.shape[:-1])
    if out is None:
        values = torch.empty(lead + [k], dtype=xs.dtype).pin_memory()
        indices = torch.empty(lead + [k], dtype=torch.int64).pin_memory()
    else:
        values, indices = out
        if list(values.shape) != lead + [k] or list(indices.shape) != lead + [k]:
            raise ValueError("out tensors have the wrong shape")
        if values.dtype != xs.dtype or indices.dtype != torch.int64 or not (
                values.is_contiguous() and indices.is_contiguous()):
            raise ValueError("out tensors must be contiguous, values in the input dtype, indices int64")
    if rows == 0 or k == 0:
        return values, indices
    lib = _native.lib()
    with torch.cuda.device(device):
        nbytes = lib.atk_topk_host_scratch_bytes(code, rows, n, k, j, k_mult, chunk_rows)
        scratch = _scratch(device, nbytes)
        # the library works on its own streams: anything torch still has queued on
        # this device (e.g. a previous user of recycled memory) must finish first
        torch.cuda.synchronize(device)
        status = lib.atk_topk_host(xs.data_ptr(), code, rows, n, n, k, j, k_mult, int(interleaved),
                                   values.data_ptr(), indices.data_ptr(), scratch.data_ptr(),
                                   scratch.numel(), chunk_rows)
    _native.check(status)
    return values, indices
