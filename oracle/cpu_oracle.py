"""ctypes front end of ``atk_oracle.c`` (test infrastructure only).

Inputs are torch CPU tensors of any element type of the reference's dispatch
(approx_topk/priority_queue_approx_topk.cu:449-453).  Each is widened exactly
to a carrier type -- float for fp32 / bf16 / fp16, double for float64, int64
for the integer types -- pushed through the scalar C restatement of the
reference's CUDA semantics (.cu:25-147) for that carrier, and the selected
values are narrowed back, which is an exact round trip.
"""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
_LIB_PATH = HERE / "libatk_oracle.so"
_lib = None

_i64p = ctypes.POINTER(ctypes.c_int64)
_i64 = ctypes.c_int64

# carrier name -> (symbol suffix, ctypes scalar, torch dtype)
_CARRIERS = {
    "f32": ("", ctypes.c_float, torch.float32),
    "f64": ("_f64", ctypes.c_double, torch.float64),
    "i64": ("_i64", ctypes.c_int64, torch.int64),
}


def carrier_of(dtype: torch.dtype) -> str:
    if dtype == torch.float64:
        return "f64"
    return "f32" if dtype.is_floating_point else "i64"


def build(force: bool = False) -> Path:
    """Compile the C oracle with the Makefile next to it."""
    newest = max((HERE / name).stat().st_mtime for name in ("atk_oracle.c", "atk_oracle_body.inc"))
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < newest:
        subprocess.run(["make", "-C", str(HERE), "-B", "libatk_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_LIB_PATH))
        for suffix, scalar, _ in _CARRIERS.values():
            ptr = ctypes.POINTER(scalar)
            f = getattr(L, "atk_oracle_stage1" + suffix)
            f.argtypes = [ptr, _i64, _i64, _i64, _i64, ctypes.c_int, ctypes.c_int, scalar, ptr, _i64p]
            f.restype = ctypes.c_int
            f = getattr(L, "atk_oracle_select" + suffix)
            f.argtypes = [ptr, _i64p, _i64, _i64, _i64, ptr, _i64p]
            f.restype = ctypes.c_int
            f = getattr(L, "atk_oracle_topk" + suffix)
            f.argtypes = [ptr, _i64, _i64, _i64, _i64, ctypes.c_int, _i64, ctypes.c_int, scalar, ptr, _i64p]
            f.restype = ctypes.c_int
            f = getattr(L, "atk_oracle_bucketed_argmax" + suffix)
            f.argtypes = [ptr, _i64, _i64, _i64, _i64, ctypes.c_int, scalar, ptr, _i64p]
            f.restype = ctypes.c_int
            f = getattr(L, "atk_oracle_recall" + suffix)
            f.argtypes = [ptr, _i64, _i64, _i64, ptr, _i64]
            f.restype = ctypes.c_double
        _lib = L
    return _lib


def _fn(name: str, dtype: torch.dtype):
    return getattr(lib(), name + _CARRIERS[carrier_of(dtype)][0])


def _fp(t: torch.Tensor):
    """Pointer to a carrier-typed tensor's data."""
    scalar = {torch.float32: ctypes.c_float, torch.float64: ctypes.c_double, torch.int64: ctypes.c_int64}[t.dtype]
    return ctypes.cast(t.data_ptr(), ctypes.POINTER(scalar))


def _ip(t: torch.Tensor):
    return ctypes.cast(t.data_ptr(), _i64p)


def _rows(x: torch.Tensor) -> tuple[torch.Tensor, tuple[int, ...]]:
    """Flatten to (rows, n) in the carrier type, contiguous on CPU; keep the batch shape."""
    if x.ndim == 0:
        x = x.reshape(1)
    batch = tuple(x.shape[:-1])
    carrier = _CARRIERS[carrier_of(x.dtype)][2]
    x2 = x.detach().to("cpu").reshape(-1, x.shape[-1]).to(carrier).contiguous()
    return x2, batch


NEG_INF = float("-inf")


def lowest(dtype: torch.dtype):
    """The reference's queue sentinel, numeric_limits<T>::lowest() (.cu:95-101)."""
    return torch.finfo(dtype).min if dtype.is_floating_point else torch.iinfo(dtype).min


def _sentinel(dtype: torch.dtype, sentinel):
    """Initial queue value in the carrier type: -inf for the float types unless
    told otherwise; the type's lowest value for the integer types (where it is
    what the reference uses too)."""
    if dtype.is_floating_point:
        return float(sentinel)
    return int(lowest(dtype))


def stage1(x: torch.Tensor, k0: int, j: int, interleaved: bool = True,
           sentinel: float = NEG_INF) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-bucket top-j of the last dim; slot layout bucket*j + q, q ascending."""
    x2, batch = _rows(x)
    rows, n = x2.shape
    vals = torch.empty((rows, k0), dtype=x2.dtype)
    idx = torch.empty((rows, k0), dtype=torch.int64)
    rc = _fn("atk_oracle_stage1", x.dtype)(_fp(x2), rows, n, n, k0, j, int(interleaved),
                                           _sentinel(x.dtype, sentinel), _fp(vals), _ip(idx))
    if rc != 0:
        raise ValueError(f"atk_oracle_stage1 rejected the arguments (rc={rc})")
    return vals.to(x.dtype).reshape(*batch, k0), idx.reshape(*batch, k0)


def select(cand_vals: torch.Tensor, cand_idx: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Exact top-k over the candidates of each row (value descending order)."""
    v2, batch = _rows(cand_vals)
    i2 = cand_idx.detach().to("cpu").reshape(-1, cand_idx.shape[-1]).contiguous()
    rows, k0 = v2.shape
    vals = torch.empty((rows, k), dtype=v2.dtype)
    idx = torch.empty((rows, k), dtype=torch.int64)
    rc = _fn("atk_oracle_select", cand_vals.dtype)(_fp(v2), _ip(i2), rows, k0, k, _fp(vals), _ip(idx))
    if rc != 0:
        raise ValueError(f"atk_oracle_select rejected the arguments (rc={rc})")
    return vals.to(cand_vals.dtype).reshape(*batch, k), idx.reshape(*batch, k)


def topk(x: torch.Tensor, k: int, j: int = 1, k_mult: int = 1, interleaved: bool = True,
         sentinel: float = NEG_INF) -> tuple[torch.Tensor, torch.Tensor]:
    """approx_topk.topk(x, k, dim=-1, j, k_mult, interleaved) on the CPU."""
    x2, batch = _rows(x)
    rows, n = x2.shape
    vals = torch.empty((rows, k), dtype=x2.dtype)
    idx = torch.empty((rows, k), dtype=torch.int64)
    rc = _fn("atk_oracle_topk", x.dtype)(_fp(x2), rows, n, n, k, j, k_mult, int(interleaved),
                                         _sentinel(x.dtype, sentinel), _fp(vals), _ip(idx))
    if rc != 0:
        raise ValueError(f"atk_oracle_topk rejected the arguments (rc={rc})")
    return vals.to(x.dtype).reshape(*batch, k), idx.reshape(*batch, k)


def bucketed_argmax(x: torch.Tensor, k: int, interleaved: bool) -> tuple[torch.Tensor, torch.Tensor]:
    """k_b = 1 path with first-max tie rule and the padded geometry of topk_torch."""
    x2, batch = _rows(x)
    rows, n = x2.shape
    vals = torch.empty((rows, k), dtype=x2.dtype)
    idx = torch.empty((rows, k), dtype=torch.int64)
    pad = lowest(x.dtype)
    rc = _fn("atk_oracle_bucketed_argmax", x.dtype)(_fp(x2), rows, n, n, k, int(interleaved), pad,
                                                    _fp(vals), _ip(idx))
    if rc != 0:
        raise ValueError(f"atk_oracle_bucketed_argmax rejected the arguments (rc={rc})")
    return vals.to(x.dtype).reshape(*batch, k), idx.reshape(*batch, k)


def scores(q: torch.Tensor, keys: torch.Tensor, scale: float) -> torch.Tensor:
    """Reference scores for the fused producer (atk_score_topk / atk_scores): q [rows, d],
    keys [rows, n, d] of a 16-bit float type; dot products in double precision, rounded to
    float, times `scale`, rounded once to the element type.  The kernels agree with it to
    within one unit in the last place."""
    rows, n, d = keys.shape
    qf = q.detach().to("cpu").float().contiguous()
    kf = keys.detach().to("cpu").float().contiguous()
    out = torch.empty(rows, n, dtype=torch.float32)
    f = lib().atk_oracle_scores
    fp = ctypes.POINTER(ctypes.c_float)
    f.argtypes = [fp, fp, _i64, _i64, _i64, ctypes.c_float, fp]
    f.restype = ctypes.c_int
    rc = f(ctypes.cast(qf.data_ptr(), fp), ctypes.cast(kf.data_ptr(), fp), rows, n, d, float(scale),
           ctypes.cast(out.data_ptr(), fp))
    if rc != 0:
        raise ValueError("atk_oracle_scores rejected the arguments")
    return out.to(q.dtype)


def recall(x: torch.Tensor, approx_vals: torch.Tensor) -> float:
    """Value-threshold recall (reference benchmarks/run_recall.py:27-36)."""
    x2, _ = _rows(x)
    a2, _ = _rows(approx_vals.to(x.dtype))
    rows, n = x2.shape
    return float(_fn("atk_oracle_recall", x.dtype)(_fp(x2), rows, n, n, _fp(a2), a2.shape[-1]))


def canonical(vals: torch.Tensor, idx: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Sort every row's (value, index) pairs by value descending, index ascending."""
    v = vals.detach().to("cpu").to(_CARRIERS[carrier_of(vals.dtype)][2]).reshape(-1, vals.shape[-1])
    i = idx.detach().to("cpu").reshape(-1, idx.shape[-1])
    o1 = torch.argsort(i, dim=-1, stable=True)
    v, i = v.gather(-1, o1), i.gather(-1, o1)
    o2 = torch.argsort(v, dim=-1, descending=True, stable=True)
    return v.gather(-1, o2), i.gather(-1, o2)
