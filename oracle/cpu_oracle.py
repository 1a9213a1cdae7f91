"""ctypes front end of ``atk_oracle.c`` (test infrastructure only).

Inputs are torch CPU tensors (fp32 / bf16 / fp16); 16-bit inputs are widened to
float exactly, pushed through the scalar C restatement of the reference's CUDA
semantics (approx_topk/priority_queue_approx_topk.cu:25-147) and the selected
values narrowed back, which is an exact round trip.
"""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
_LIB_PATH = HERE / "libatk_oracle.so"
_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)
_i64p = ctypes.POINTER(ctypes.c_int64)
_i64 = ctypes.c_int64


def build(force: bool = False) -> Path:
    """Compile the C oracle with the Makefile next to it."""
    src = HERE / "atk_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B", "libatk_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_LIB_PATH))
        L.atk_oracle_stage1.argtypes = [_f32p, _i64, _i64, _i64, _i64, ctypes.c_int, ctypes.c_int,
                                        ctypes.c_float, _f32p, _i64p]
        L.atk_oracle_stage1.restype = ctypes.c_int
        L.atk_oracle_select.argtypes = [_f32p, _i64p, _i64, _i64, _i64, _f32p, _i64p]
        L.atk_oracle_select.restype = ctypes.c_int
        L.atk_oracle_topk.argtypes = [_f32p, _i64, _i64, _i64, _i64, ctypes.c_int, _i64, ctypes.c_int,
                                      ctypes.c_float, _f32p, _i64p]
        L.atk_oracle_topk.restype = ctypes.c_int
        L.atk_oracle_bucketed_argmax.argtypes = [_f32p, _i64, _i64, _i64, _i64, ctypes.c_int,
                                                 ctypes.c_float, _f32p, _i64p]
        L.atk_oracle_bucketed_argmax.restype = ctypes.c_int
        L.atk_oracle_recall.argtypes = [_f32p, _i64, _i64, _i64, _f32p, _i64]
        L.atk_oracle_recall.restype = ctypes.c_double
        _lib = L
    return _lib


def _fp(t: torch.Tensor):
    return ctypes.cast(t.data_ptr(), _f32p)


def _ip(t: torch.Tensor):
    return ctypes.cast(t.data_ptr(), _i64p)


def _rows(x: torch.Tensor) -> tuple[torch.Tensor, tuple[int, ...]]:
    """Flatten to (rows, n) float32 contiguous on CPU; keep the batch shape."""
    if x.ndim == 0:
        x = x.reshape(1)
    batch = tuple(x.shape[:-1])
    x2 = x.detach().to("cpu").reshape(-1, x.shape[-1]).to(torch.float32).contiguous()
    return x2, batch


NEG_INF = float("-inf")


def lowest(dtype: torch.dtype) -> float:
    """The reference's queue sentinel, numeric_limits<T>::lowest() (.cu:95-101)."""
    return torch.finfo(dtype).min


def stage1(x: torch.Tensor, k0: int, j: int, interleaved: bool = True,
           sentinel: float = NEG_INF) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-bucket top-j of the last dim; slot layout bucket*j + q, q ascending."""
    x2, batch = _rows(x)
    rows, n = x2.shape
    vals = torch.empty((rows, k0), dtype=torch.float32)
    idx = torch.empty((rows, k0), dtype=torch.int64)
    rc = lib().atk_oracle_stage1(_fp(x2), rows, n, n, k0, j, int(interleaved), sentinel,
                                 _fp(vals), _ip(idx))
    if rc != 0:
        raise ValueError(f"atk_oracle_stage1 rejected the arguments (rc={rc})")
    return vals.to(x.dtype).reshape(*batch, k0), idx.reshape(*batch, k0)


def select(cand_vals: torch.Tensor, cand_idx: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Exact top-k over the candidates of each row (value descending order)."""
    v2, batch = _rows(cand_vals)
    i2 = cand_idx.detach().to("cpu").reshape(-1, cand_idx.shape[-1]).contiguous()
    rows, k0 = v2.shape
    vals = torch.empty((rows, k), dtype=torch.float32)
    idx = torch.empty((rows, k), dtype=torch.int64)
    rc = lib().atk_oracle_select(_fp(v2), _ip(i2), rows, k0, k, _fp(vals), _ip(idx))
    if rc != 0:
        raise ValueError(f"atk_oracle_select rejected the arguments (rc={rc})")
    return vals.to(cand_vals.dtype).reshape(*batch, k), idx.reshape(*batch, k)


def topk(x: torch.Tensor, k: int, j: int = 1, k_mult: int = 1, interleaved: bool = True,
         sentinel: float = NEG_INF) -> tuple[torch.Tensor, torch.Tensor]:
    """approx_topk.topk(x, k, dim=-1, j, k_mult, interleaved) on the CPU."""
    x2, batch = _rows(x)
    rows, n = x2.shape
    vals = torch.empty((rows, k), dtype=torch.float32)
    idx = torch.empty((rows, k), dtype=torch.int64)
    rc = lib().atk_oracle_topk(_fp(x2), rows, n, n, k, j, k_mult, int(interleaved), sentinel,
                               _fp(vals), _ip(idx))
    if rc != 0:
        raise ValueError(f"atk_oracle_topk rejected the arguments (rc={rc})")
    return vals.to(x.dtype).reshape(*batch, k), idx.reshape(*batch, k)


def bucketed_argmax(x: torch.Tensor, k: int, interleaved: bool) -> tuple[torch.Tensor, torch.Tensor]:
    """k_b = 1 path with first-max tie rule and the padded geometry of topk_torch."""
    x2, batch = _rows(x)
    rows, n = x2.shape
    vals = torch.empty((rows, k), dtype=torch.float32)
    idx = torch.empty((rows, k), dtype=torch.int64)
    pad = torch.finfo(x.dtype).min if x.dtype.is_floating_point else float(torch.iinfo(x.dtype).min)
    rc = lib().atk_oracle_bucketed_argmax(_fp(x2), rows, n, n, k, int(interleaved), pad,
                                          _fp(vals), _ip(idx))
    if rc != 0:
        raise ValueError(f"atk_oracle_bucketed_argmax rejected the arguments (rc={rc})")
    return vals.to(x.dtype).reshape(*batch, k), idx.reshape(*batch, k)


def recall(x: torch.Tensor, approx_vals: torch.Tensor) -> float:
    """Value-threshold recall (reference benchmarks/run_recall.py:27-36)."""
    x2, _ = _rows(x)
    a2, _ = _rows(approx_vals)
    rows, n = x2.shape
    return float(lib().atk_oracle_recall(_fp(x2), rows, n, n, _fp(a2), a2.shape[-1]))


def canonical(vals: torch.Tensor, idx: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Sort every row's (value, index) pairs by value descending, index ascending."""
    v = vals.detach().to("cpu").to(torch.float32).reshape(-1, vals.shape[-1])
    i = idx.detach().to("cpu").reshape(-1, idx.shape[-1])
    o1 = torch.argsort(i, dim=-1, stable=True)
    v, i = v.gather(-1, o1), i.gather(-1, o1)
    o2 = torch.argsort(v, dim=-1, descending=True, stable=True)
    return v.gather(-1, o2), i.gather(-1, o2)
