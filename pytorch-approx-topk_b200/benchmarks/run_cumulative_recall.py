"""Cumulative recall of the approximate operator.

Cumulative recall at i is the probability that the operator returns ALL of the
true top-i elements; with both results sorted descending that is the share of
rows whose i-th value equals the exact i-th value.  Same experiment as the
reference's (reference benchmarks/run_cumulative_recall.py:19-45): n = 16*32*40,
uniform and log-normal rows, k = n/8 and n/16, exact top-k and the operator
with 1, 2 and 4 survivors per bucket.  Writes one JSON line per (distribution,
k, method) holding the whole curve, and prints where each curve falls below 0.99,
0.9 and 0.5.

    python benchmarks/run_cumulative_recall.py --out results/cumulative_recall.jsonl
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path
from typing import Callable

import torch
from torch import Tensor

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from run_recall import N, distributions, methods  # noqa: E402

K_RATIOS = (8, 16)


def cumulative_recall(xs: Tensor, method: Callable[..., tuple[Tensor, Tensor]], k: int) -> list[float]:
    truth, _ = torch.topk(xs, k, dim=-1, sorted=True)
    got, _ = method(xs, k, dim=-1)
    got = got.sort(dim=-1, descending=True).values
    return (truth == got).float().mean(dim=0).tolist()


def first_below(curve: list[float], level: float) -> int:
    """Smallest i (1-based) with curve[i-1] < level, or len(curve) + 1 if none."""
    for i, c in enumerate(curve, 1):
        if c < level:
            return i
    return len(curve) + 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", type=Path, default=Path("results/cumulative_recall.jsonl"))
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    gen = torch.Generator(device="cuda").manual_seed(args.seed)
    args.out.parent.mkdir(parents=True, exist_ok=True)
    print(f"{'distribution':12s} {'k':>6s} {'method':14s} {'<0.99 at':>9s} {'<0.9 at':>8s} {'<0.5 at':>8s}")
    with args.out.open("w") as f:
        for dist_name, draw in distributions(gen).items():
            for ratio in K_RATIOS:
                k = N // ratio
                for method_name, method in methods().items():
                    curve = cumulative_recall(draw(), method, k)
                    print(json.dumps(dict(distribution=dist_name, method=method_name, n=N, k=k,
                                          cumulative_recall=curve)), file=f)
                    print(f"{dist_name:12s} {k:6d} {method_name:14s} {first_below(curve, 0.99):9d} "
                          f"{first_below(curve, 0.9):8d} {first_below(curve, 0.5):8d}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
