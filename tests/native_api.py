"""Thin torch-tensor wrappers over the C ABI for the GPU tests (test infrastructure).

They call exactly the `extern "C"` entry points of include/atk.h through
ctypes, with device pointers and the current stream.
"""

from __future__ import annotations

import torch

from approx_topk import _native


def _stream(x):
    return torch.cuda.current_stream(x.device).cuda_stream


def stage1(x: torch.Tensor, k0: int, j: int, interleaved: bool = True, mode: int = -1, use_workspace: bool = True):
    assert x.is_cuda and x.ndim == 2 and x.stride(1) == 1
    rows, n = x.shape
    vals = torch.empty((rows, k0), device=x.device, dtype=x.dtype)
    idx = torch.empty((rows, k0), device=x.device, dtype=torch.int64)
    lib = _native.lib()
    code = _native.dtype_code(x.dtype)
    ws_bytes = lib.atk_stage1_workspace_bytes(code, rows, n, k0, j, int(interleaved)) if use_workspace else 0
    ws = torch.empty(max(ws_bytes, 1), device=x.device, dtype=torch.uint8)
    rc = lib.atk_stage1(x.data_ptr(), code, rows, n, x.stride(0), k0, j, int(interleaved), mode,
                        vals.data_ptr(), idx.data_ptr(), k0, ws.data_ptr() if ws_bytes else None, ws_bytes, _stream(x))
    _native.check(rc)
    return vals, idx


def stage1_slab(slab: torch.Tensor, total_buckets: int, col_offset: int, j: int):
    assert slab.is_cuda and slab.ndim == 2 and slab.is_contiguous()
    stripes, cols = slab.shape
    vals = torch.empty((cols * j,), device=slab.device, dtype=slab.dtype)
    idx = torch.empty((cols * j,), device=slab.device, dtype=torch.int64)
    lib = _native.lib()
    code = _native.dtype_code(slab.dtype)
    ws_bytes = lib.atk_stage1_slab_workspace_bytes(code, stripes, cols, j)
    ws = torch.empty(max(ws_bytes, 1), device=slab.device, dtype=torch.uint8)
    rc = lib.atk_stage1_slab(slab.data_ptr(), code, stripes, cols, total_buckets, col_offset, j,
                             vals.data_ptr(), idx.data_ptr(), ws.data_ptr() if ws_bytes else None, ws_bytes,
                             _stream(slab))
    _native.check(rc)
    return vals, idx


def select(cand_vals: torch.Tensor, cand_idx: torch.Tensor, k: int):
    assert cand_vals.is_cuda and cand_vals.ndim == 2 and cand_vals.is_contiguous()
    rows, k0 = cand_vals.shape
    code = _native.dtype_code(cand_vals.dtype)
    lib = _native.lib()
    ws_bytes = lib.atk_select_workspace_bytes(code, rows, k0, k)
    ws = torch.empty(max(ws_bytes, 1), device=cand_vals.device, dtype=torch.uint8)
    vals = torch.empty((rows, k), device=cand_vals.device, dtype=cand_vals.dtype)
    idx = torch.empty((rows, k), device=cand_vals.device, dtype=torch.int64)
    rc = lib.atk_select(cand_vals.data_ptr(), cand_idx.data_ptr(), code, rows, k0, k0, k,
                        vals.data_ptr(), idx.data_ptr(), k, ws.data_ptr() if ws_bytes else None, ws_bytes,
                        _stream(cand_vals))
    _native.check(rc)
    return vals, idx


def topk(x: torch.Tensor, k: int, j: int, k_mult: int, interleaved: bool = True):
    assert x.is_cuda and x.ndim == 2 and x.stride(1) == 1
    rows, n = x.shape
    code = _native.dtype_code(x.dtype)
    lib = _native.lib()
    ws_bytes = lib.atk_topk_workspace_bytes(code, rows, n, k, j, k_mult)
    ws = torch.empty(max(ws_bytes, 1), device=x.device, dtype=torch.uint8)
    vals = torch.empty((rows, k), device=x.device, dtype=x.dtype)
    idx = torch.empty((rows, k), device=x.device, dtype=torch.int64)
    rc = lib.atk_topk(x.data_ptr(), code, rows, n, x.stride(0), k, j, k_mult, int(interleaved), -1,
                      vals.data_ptr(), idx.data_ptr(), k, ws.data_ptr() if ws_bytes else None, ws_bytes,
                      _stream(x))
    _native.check(rc)
    return vals, idx


def bucketed_argmax(x: torch.Tensor, k: int, interleaved: bool):
    assert x.is_cuda and x.ndim == 2 and x.stride(1) == 1
    rows, n = x.shape
    vals = torch.empty((rows, k), device=x.device, dtype=x.dtype)
    idx = torch.empty((rows, k), device=x.device, dtype=torch.int64)
    lib = _native.lib()
    code = _native.dtype_code(x.dtype)
    ws_bytes = lib.atk_stage1_workspace_bytes(code, rows, n, k, 1, int(interleaved)) if k <= n else 0
    ws = torch.empty(max(ws_bytes, 1), device=x.device, dtype=torch.uint8)
    rc = lib.atk_bucketed_argmax(x.data_ptr(), code, rows, n, x.stride(0), k, int(interleaved), vals.data_ptr(),
                                 idx.data_ptr(), k, ws.data_ptr() if ws_bytes else None, ws_bytes, _stream(x))
    _native.check(rc)
    return vals, idx


def topk_host(x_host: torch.Tensor, k: int, j: int, k_mult: int, interleaved: bool = True,
              chunk_rows: int = 0, device: str = "cuda"):
    """Host buffers in, host buffers out (pinned for speed); device scratch from torch."""
    assert not x_host.is_cuda and x_host.ndim == 2 and x_host.is_contiguous()
    rows, n = x_host.shape
    code = _native.dtype_code(x_host.dtype)
    lib = _native.lib()
    sbytes = lib.atk_topk_host_scratch_bytes(code, rows, n, k, j, k_mult, chunk_rows)
    scratch = torch.empty(max(sbytes, 1), device=device, dtype=torch.uint8)
    vals = torch.empty((rows, k), dtype=x_host.dtype).pin_memory()
    idx = torch.empty((rows, k), dtype=torch.int64).pin_memory()
    with torch.cuda.device(scratch.device):
        rc = lib.atk_topk_host(x_host.data_ptr(), code, rows, n, n, k, j, k_mult, int(interleaved),
                               vals.data_ptr(), idx.data_ptr(), scratch.data_ptr(), sbytes, chunk_rows)
    _native.check(rc)
    return vals, idx
