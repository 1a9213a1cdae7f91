"""Top-50 and top-k recall of the approximate operator as k grows.

Same experiment as the reference's (reference benchmarks/run_recall.py:15-39):
rows of n = 16*32*40 samples, uniform and log-normal, 100 rows each; for every
k in 1024, 1152, ... < n the exact top-k and the operator with 1, 2 and 4
survivors per bucket; recall is value-threshold based, so ties cannot hurt it:
the share of returned values at least as large as the true 50th (top-50) or
k-th (top-k) largest.  Results go to a JSONL file (one line per distribution,
method and k) and a short table on stdout; with matplotlib installed, ``--plot``
also draws the reference's figure.

    python benchmarks/run_recall.py --out results/recall.jsonl [--step 1024] [--plot]
"""

from __future__ import annotations

import argparse
import json
import sys
from functools import partial
from pathlib import Path
from typing import Callable

import torch
from torch import Tensor

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from approx_topk import priority_queue  # noqa: E402

N_REPEATS = 100
N = 16 * 32 * 40


def distributions(gen: torch.Generator) -> dict[str, Callable[[], Tensor]]:
    return {
        "uniform": lambda: torch.rand(N_REPEATS, N, generator=gen, device="cuda"),
        "log normal": lambda: torch.randn(N_REPEATS, N, generator=gen, device="cuda").exp(),
    }


def methods() -> dict[str, Callable[..., tuple[Tensor, Tensor]]]:
    out: dict[str, Callable[..., tuple[Tensor, Tensor]]] = {"exact": torch.topk}
    for per_bucket in (1, 2, 4):
        out[f"{per_bucket} per bucket"] = partial(priority_queue.topk, j=per_bucket)
    return out


def recall_pair(xs: Tensor, method: Callable[..., tuple[Tensor, Tensor]], k: int) -> tuple[float, float]:
    """(top-50 recall, top-k recall) averaged over the rows of ``xs``."""
    truth, _ = torch.topk(xs, k, dim=-1, sorted=True)
    got, _ = method(xs, k, dim=-1)
    top_50 = (got >= truth[:, 49:50]).sum(-1).float().div(50).mean().item()
    top_k = (got >= truth[:, k - 1:k]).sum(-1).float().div(k).mean().item()
    return top_50, top_k


def valid_ks(step: int) -> list[int]:
    # the operator needs j | k for j in {1, 2, 4}; the reference's ks (multiples of 128) all qualify
    return [k for k in range(1024, N, step) if k % 4 == 0]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", type=Path, default=Path("results/recall.jsonl"))
    ap.add_argument("--step", type=int, default=128, help="spacing of the k values (reference: 128)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--plot", action="store_true")
    args = ap.parse_args(argv)
    gen = torch.Generator(device="cuda").manual_seed(args.seed)
    rows = []
    for dist_name, draw in distributions(gen).items():
        for method_name, method in methods().items():
            for k in valid_ks(args.step):
                top_50, top_k = recall_pair(draw(), method, k)
                rows.append(dict(distribution=dist_name, method=method_name, n=N, k=k,
                                 top_50_recall=top_50, top_k_recall=top_k))
    args.out.parent.mkdir(parents=True, exist_ok=True)
    with args.out.open("w") as f:
        for r in rows:
            print(json.dumps(r), file=f)
    ks = valid_ks(args.step)
    probe = [ks[0], ks[len(ks) // 2], ks[-1]]
    print(f"{'distribution':12s} {'method':14s} " + " ".join(f"top-k@{k:<6d}" for k in probe))
    for dist_name in ("uniform", "log normal"):
        for method_name in methods():
            vals = {r["k"]: r["top_k_recall"] for r in rows
                    if r["distribution"] == dist_name and r["method"] == method_name}
            print(f"{dist_name:12s} {method_name:14s} " + " ".join(f"{vals[k]:<12.4f}" for k in probe))
    if args.plot:
        draw_figure(rows, args.out.with_suffix(".png"))
    return 0


def draw_figure(rows: list[dict], path: Path) -> None:
    try:
        import matplotlib.pyplot as plt
    except ImportError:
        print("matplotlib is not installed: no figure written", file=sys.stderr)
        return
    dists = sorted({r["distribution"] for r in rows})
    fig, axes = plt.subplots(len(dists), 2, figsize=(10, 10), squeeze=False, sharex="col", sharey=True)
    for ax_row, dist in zip(axes, dists):
        ax_row[0].set_ylabel(dist)
        for name in sorted({r["method"] for r in rows}):
            sel = [r for r in rows if r["distribution"] == dist and r["method"] == name]
            ax_row[0].plot([r["k"] for r in sel], [r["top_50_recall"] for r in sel], label=name)
            ax_row[1].plot([r["k"] for r in sel], [r["top_k_recall"] for r in sel], label=name)
    axes[0, 0].legend()
    axes[0, 0].set_title("top 50 recall")
    axes[0, 1].set_title("top k recall")
    for ax in axes[-1]:
        ax.set_xlabel("k")
    fig.tight_layout()
    fig.savefig(path)


if __name__ == "__main__":
    sys.exit(main())
