"""Generate golden vectors by running the reference's own Python (CPU) code.

Run from the repository root, with the reference checkout available:

    python tests/golden/make_golden.py --reference-root <path to the reference checkout>

The script puts ONLY the reference on ``sys.path`` (never this repository's
package), imports ``approx_topk.experimental.autobucket.bucketed_torch_topk`` and
``approx_topk.experimental.bucketed_argmax.topk_torch`` from it unmodified, runs
them on small seeded CPU inputs and stores inputs plus outputs in
``tests/golden/reference_cpu_vectors.npz``.  The fixture travels with the
repository; the reference checkout does not need to exist where tests run.

Stored per case (prefix ``c<i>_``): ``x`` (float32; 16-bit inputs are stored
widened, which is exact), ``values`` and ``indices`` each sorted ascending along
the last axis (order inside the reference's output is not part of its
contract), and a JSON header with the call arguments.

A second file, ``reference_cpu_vectors_all_dtypes.npz``, holds the same kind of
cases for the other element types of the reference's native dispatch (float64,
int64, int32, int16, int8, uint8), with ``x`` and ``values`` stored in the
element type itself.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
OUT = HERE / "reference_cpu_vectors.npz"
OUT_WIDE = HERE / "reference_cpu_vectors_all_dtypes.npz"

WIDE_DTYPES = {"float64": torch.float64, "int64": torch.int64, "int32": torch.int32,
               "int16": torch.int16, "int8": torch.int8, "uint8": torch.uint8}

DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def cases():
    out = []
    # (rows, n, k, j, k_mult, interleaved, dtype, distribution)
    for interleaved in (True, False):
        for j in (1, 2, 4):
            out.append((3, 512, 64, j, 1, interleaved, "float32", "randn"))
            out.append((2, 1001, 12 * j, j, 1, interleaved, "float32", "randn"))     # b does not divide n
            out.append((2, 1000, 16, j, 4, interleaved, "float32", "randn"))         # stage 2
        out.append((2, 17, 8, 2, 1, interleaved, "float32", "randn"))
        out.append((4, 2048, 256, 4, 2, interleaved, "bfloat16", "randn"))
        out.append((4, 4000, 64, 2, 4, interleaved, "float16", "randn"))
        out.append((2, 3000, 30, 3, 1, interleaved, "float32", "randn"))             # j = 3
        out.append((2, 4096, 64, 1, 1, interleaved, "float32", "linspace"))          # correlated rows
    return out


def make_input(rows, n, dtype, dist, seed):
    g = torch.Generator().manual_seed(seed)
    if dist == "randn":
        x = torch.randn(rows, n, generator=g)
    else:
        x = torch.linspace(0, 1, n)[None, :] + 0.01 * torch.randn(rows, n, generator=g)
    return x.to(DTYPES[dtype])


def make_wide_input(rows, n, dtype, seed):
    """Seeded input of one of the wider dispatch types: the full value range,
    with the type's extreme values planted so that the sentinel handling shows."""
    g = torch.Generator().manual_seed(seed)
    t = WIDE_DTYPES[dtype]
    if t == torch.float64:
        x = torch.randn(rows, n, generator=g, dtype=torch.float64) * 1e100
    else:
        info = torch.iinfo(t)
        if t == torch.int64:
            hi = torch.randint(-2**31, 2**31, (rows, n), generator=g, dtype=torch.int64)
            lo = torch.randint(0, 2**32, (rows, n), generator=g, dtype=torch.int64)
            x = hi * 2**32 + lo
        else:
            x = torch.randint(info.min, info.max + 1, (rows, n), generator=g, dtype=torch.int64).to(t)
        x[:, 3] = info.min
        x[:, n // 2] = info.max
        x[:, n - 1] = info.min
    return x


def wide_cases():
    out = []
    for dtype in WIDE_DTYPES:
        for interleaved in (True, False):
            for j in (1, 2, 3, 4):
                out.append((2, 1001, 12 * j, j, 1, interleaved, dtype))     # b does not divide n
            out.append((2, 1000, 16, 2, 4, interleaved, dtype))             # stage 2
            out.append((1, 300, 296, 4, 1, interleaved, dtype))             # buckets of 4 or 5 elements
    return out


def write_wide(bucketed_torch_topk, topk_torch) -> None:
    store: dict[str, np.ndarray] = {}
    meta = []
    for i, (rows, n, k, j, k_mult, interleaved, dtype) in enumerate(wide_cases()):
        x = make_wide_input(rows, n, dtype, seed=3000 + i)
        v, idx = bucketed_torch_topk(x, k=k, dim=-1, k_mult=k_mult, k_per_bucket=j, interleaved=interleaved)
        store[f"c{i}_x"] = x.numpy()
        store[f"c{i}_values"] = v.sort(dim=-1).values.numpy()
        store[f"c{i}_indices"] = idx.sort(dim=-1).values.numpy()
        meta.append(dict(kind="bucketed_torch_topk", rows=rows, n=n, k=k, j=j, k_mult=k_mult,
                         interleaved=interleaved, dtype=dtype))
    base = len(meta)
    t = 0
    for dtype in WIDE_DTYPES:
        for rows, n, k in ((2, 1000, 64), (2, 37, 5)):
            for interleaved in (True, False):
                i = base + t
                t += 1
                x = make_wide_input(rows, n, dtype, seed=4000 + i)
                v, idx = topk_torch(x, k=k, dim=-1, interleaved=interleaved)
                store[f"c{i}_x"] = x.numpy()
                store[f"c{i}_values"] = v.numpy()
                store[f"c{i}_indices"] = idx.numpy()
                meta.append(dict(kind="topk_torch", rows=rows, n=n, k=k, interleaved=interleaved, dtype=dtype))
    store["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(OUT_WIDE, **store)
    print(f"wrote {OUT_WIDE} ({OUT_WIDE.stat().st_size} bytes, {len(meta)} cases)")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-root", default=os.environ.get("ATK_REFERENCE_ROOT"))
    args = ap.parse_args()
    if not args.reference_root:
        ap.error("--reference-root (or ATK_REFERENCE_ROOT) is required")
    sys.path.insert(0, str(Path(args.reference_root).resolve()))
    from approx_topk.experimental.autobucket import bucketed_torch_topk  # the reference's
    from approx_topk.experimental.bucketed_argmax import topk_torch      # the reference's
    import approx_topk
    assert Path(approx_topk.__file__).resolve().is_relative_to(Path(args.reference_root).resolve())

    store: dict[str, np.ndarray] = {}
    meta = []
    for i, (rows, n, k, j, k_mult, interleaved, dtype, dist) in enumerate(cases()):
        x = make_input(rows, n, dtype, dist, seed=1000 + i)
        v, idx = bucketed_torch_topk(x, k=k, dim=-1, k_mult=k_mult, k_per_bucket=j, interleaved=interleaved)
        store[f"c{i}_x"] = x.float().numpy()
        store[f"c{i}_values"] = v.float().sort(dim=-1).values.numpy()
        store[f"c{i}_indices"] = idx.sort(dim=-1).values.numpy()
        meta.append(dict(kind="bucketed_torch_topk", rows=rows, n=n, k=k, j=j, k_mult=k_mult,
                         interleaved=interleaved, dtype=dtype, dist=dist))
    base = len(meta)
    # k_b = 1 arg-max (bucket order is part of this contract: stored unsorted)
    argmax_cases = [(2, 20, 3, "float32"), (3, 1000, 7, "float32"), (2, 4096, 256, "float32"),
                    (2, 1000, 64, "float16"), (2, 1000, 64, "bfloat16"), (1, 10, 4, "float32")]
    for t, (rows, n, k, dtype) in enumerate(argmax_cases):
        for interleaved in (True, False):
            i = base + 2 * t + int(not interleaved)
            x = make_input(rows, n, dtype, "randn", seed=2000 + i)
            v, idx = topk_torch(x, k=k, dim=-1, interleaved=interleaved)
            store[f"c{i}_x"] = x.float().numpy()
            store[f"c{i}_values"] = v.float().numpy()
            store[f"c{i}_indices"] = idx.numpy()
            meta.append(dict(kind="topk_torch", rows=rows, n=n, k=k, interleaved=interleaved, dtype=dtype))
    # metadata is sorted by case number
    store["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(OUT, **store)
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes, {len(meta)} cases)")
    write_wide(bucketed_torch_topk, topk_torch)
    return 0


if __name__ == "__main__":
    sys.exit(main())
