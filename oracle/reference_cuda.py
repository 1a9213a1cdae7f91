"""Loader for the reference's own CUDA operator (TEST / BASELINE INFRASTRUCTURE ONLY;
the product never imports this).

``oracle/build_ref.py`` compiles the reference's CUDA file, unmodified and in
place, into ``oracle/_ref/atk_reference_cuda.so``.  The GPU parity tests compare
the new kernels with it on the same inputs, and ``bench.py`` times it as the
"reference CUDA kernel on the same GPU" baseline beside its own numbers.
"""

from __future__ import annotations

import importlib.util
from functools import cache
from pathlib import Path

import torch

SO_PATH = Path(__file__).resolve().parent / "_ref" / "atk_reference_cuda.so"


@cache
def module():
    if not SO_PATH.exists():
        return None
    spec = importlib.util.spec_from_file_location("atk_reference_cuda", SO_PATH)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def available() -> bool:
    return module() is not None


def reference_topk(xs, k, dim=-1, j=1, k_mult=1, interleaved=True, multithread_buckets=False):
    """What the reference's Python wrapper does around its kernel
    (approx_topk/priority_queue.py:51-88): allocate k*k_mult candidates, run the
    kernel, then torch.topk(sorted=False) + gather when k_mult > 1."""
    mod = module()
    dim = dim % xs.ndim
    k0 = k * k_mult
    shape = list(xs.shape)
    shape[dim] = k0
    vals = torch.empty(shape, device=xs.device, dtype=xs.dtype)
    idx = torch.empty(shape, device=xs.device, dtype=torch.int64)
    mod.PriorityQueueTopK(xs, k0, j, dim, True, interleaved, multithread_buckets, vals, idx)
    if k0 == k:
        return vals, idx
    v2, i2 = torch.topk(vals, k, dim, True, sorted=False)
    return v2, idx.gather(dim, i2)


def reference_stage1(xs, k0, j, interleaved=True, multithread_buckets=False):
    return reference_topk(xs, k0, -1, j, 1, interleaved, multithread_buckets)
