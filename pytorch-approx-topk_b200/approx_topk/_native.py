"""ctypes binding of ``libatk.so`` — the C-ABI library holding the sm_100a kernels.

This module is the only place where Python meets native code.  There is no
fallback of any kind: if the library is missing, cannot be loaded or the device
is not an sm_100 part, the call fails with an error that says so.
"""

from __future__ import annotations

import ctypes
import os
from functools import cache
from pathlib import Path

import torch

_LIB_ENV = "ATK_LIBRARY"
_DEFAULT_LIB = Path(__file__).resolve().parent / "lib" / "libatk.so"

ATK_OK = 0
ATK_ERR_BAD_J = -1
ATK_ERR_J_DIVIDES_K = -2
ATK_ERR_K_TOO_LARGE = -3
ATK_ERR_BAD_DTYPE = -4
ATK_ERR_BAD_ARG = -5
ATK_ERR_WORKSPACE = -6
ATK_ERR_TOO_LARGE = -7
ATK_ERR_CUDA = -8
ATK_ERR_SCRATCH_LIMIT = -9

# output formats of atk_topk_ex
ATK_OUT_I64 = 0
ATK_OUT_I32 = 1
ATK_OUT_REC32 = 2

# Codes of include/atk.h; the nine element types of the reference's native
# dispatch (approx_topk/priority_queue_approx_topk.cu:449-453).
DTYPE_CODES = {
    torch.float32: 0, torch.float16: 1, torch.bfloat16: 2,
    torch.float64: 3, torch.int32: 4, torch.int64: 5, torch.int16: 6, torch.int8: 7, torch.uint8: 8,
}

_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_int = ctypes.c_int
_sz = ctypes.c_size_t

# name -> (restype, argtypes); mirrors include/atk.h one to one.
SIGNATURES = {
    "atk_version": (_int, []),
    "atk_strerror": (ctypes.c_char_p, [_int]),
    "atk_device_supported": (_int, []),
    "atk_stage1_workspace_bytes": (_sz, [_int, _i64, _i64, _i64, _int, _int]),
    "atk_stage1": (_int, [_vp, _int, _i64, _i64, _i64, _i64, _int, _int, _int, _vp, _vp, _i64, _vp, _sz, _vp]),
    "atk_stage1_slab_workspace_bytes": (_sz, [_int, _i64, _i64, _int]),
    "atk_stage1_slab": (_int, [_vp, _int, _i64, _i64, _i64, _i64, _int, _vp, _vp, _vp, _sz, _vp]),
    "atk_select_workspace_bytes": (_sz, [_int, _i64, _i64, _i64]),
    "atk_select": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _i64, _vp, _vp, _i64, _vp, _sz, _vp]),
    "atk_select_static": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _i64, _vp, _vp, _i64, _vp]),
    "atk_topk_workspace_bytes": (_sz, [_int, _i64, _i64, _i64, _int, _i64]),
    "atk_topk": (_int, [_vp, _int, _i64, _i64, _i64, _i64, _int, _i64, _int, _int, _vp, _vp, _i64, _vp, _sz, _vp]),
    "atk_topk_ex": (_int, [_vp, _int, _i64, _i64, _i64, _i64, _int, _i64, _int, _int, _int, _vp, _vp, _i64, _vp, _sz,
                           _vp]),
    "atk_scores": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _i64, _i64, ctypes.c_float, _vp, _i64, _vp]),
    "atk_score_topk_workspace_bytes": (_sz, [_int, _i64, _i64, _i64, _int, _i64]),
    "atk_score_topk": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _i64, _i64, ctypes.c_float, _i64, _int, _i64, _vp, _vp,
                              _i64, _vp, _sz, _vp]),
    "atk_bucketed_argmax": (_int, [_vp, _int, _i64, _i64, _i64, _i64, _int, _vp, _vp, _i64, _vp, _sz, _vp]),
    "atk_topk_host_scratch_bytes": (_sz, [_int, _i64, _i64, _i64, _int, _i64, _i64]),
    "atk_topk_host": (_int, [_vp, _int, _i64, _i64, _i64, _i64, _int, _i64, _int, _vp, _vp, _vp, _sz, _i64]),
    "atk_gather_records": (_int, [_vp, _i64, _i64, _i64, _i64, _vp, _i64, _i64, _vp, _vp]),
    "atk_push_blocks": (_int, [_int, _vp, _vp, _int, _vp, _vp]),
    "atk_peer_alloc": (_int, [_sz, _vp, _vp]),
    "atk_peer_open": (_int, [_vp, _vp]),
    "atk_peer_close": (_int, [_vp]),
    "atk_peer_free": (_int, [_vp]),
    "atk_launch_count": (_i64, []),
    "atk_reset_launch_count": (None, []),
}


def library_path() -> Path:
    return Path(os.environ[_LIB_ENV]) if os.environ.get(_LIB_ENV) else _DEFAULT_LIB


@cache
def lib() -> ctypes.CDLL:
    """Load libatk.so once and attach the prototypes of every exported symbol."""
    path = library_path()
    if not path.exists():
        raise RuntimeError(
            f"approx_topk: native library {path} not found. Build it with "
            f"`python {Path(__file__).resolve().parents[1] / 'build.py'}` (needs nvcc); "
            "there is no non-CUDA fallback."
        )
    handle = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    return handle


def strerror(status: int) -> str:
    return lib().atk_strerror(status).decode()


def check(status: int) -> None:
    """Raise the exception type the reference raises for the same condition
    (its TORCH_CHECKs surface as RuntimeError)."""
    if status == ATK_OK:
        return
    msg = strerror(status)
    if status == ATK_ERR_CUDA:
        msg += f" ({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no CUDA device'})"
    raise RuntimeError(msg)


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODES[dtype]
    except KeyError:
        raise RuntimeError(
            f"approx_topk: dtype {dtype} is not supported "
            "(float32/16, bfloat16, float64, int8/16/32/64 and uint8 are)"
        ) from None


def require_cuda(xs: torch.Tensor) -> None:
    if not xs.is_cuda:
        raise RuntimeError(
            "approx_topk: expected a CUDA tensor; this build runs only on sm_100 GPUs and has no CPU path"
        )


@cache
def _device_ok(index: int) -> bool:
    with torch.cuda.device(index):
        return lib().atk_device_supported() == ATK_OK


def require_device(device: torch.device) -> None:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if not _device_ok(idx):
        raise RuntimeError(
            f"approx_topk: device cuda:{idx} ({torch.cuda.get_device_name(idx)}) is not an sm_100 GPU; "
            "libatk.so carries sm_100a code only"
        )


def current_stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def as_rows(x: torch.Tensor) -> tuple[torch.Tensor, int, int, int]:
    """View `x` (top-k axis last) as `rows` rows of length n that are `row_stride`
    elements apart, copying only when the layout cannot be described that way."""
    n = x.shape[-1]
    rows = x.numel() // n if n > 0 else 0
    if x.ndim == 1:
        if x.stride(0) != 1 and n > 1:
            x = x.contiguous()
        return x, 1, n, n
    if x.ndim == 2 and (x.stride(1) == 1 or n == 1) and (x.stride(0) >= n or rows <= 1):
        return x, rows, n, (x.stride(0) if rows > 1 else n)
    if not x.is_contiguous():
        x = x.contiguous()
    return x, rows, n, n
