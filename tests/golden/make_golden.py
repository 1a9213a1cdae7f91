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
    return 0


if __name__ == "__main__":
    sys.exit(main())
