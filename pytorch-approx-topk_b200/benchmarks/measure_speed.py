"""Runtime sweep of exact and approximate top-k on one GPU.

Writes one JSON object per line with the record layout of the reference's sweep
(reference benchmarks/measure_speed.py:27-41 for the fields, :236-255 for the
line format), so that logs of both can be loaded into one table
(``bandwidth_table.py``) or fed to the reference's own plotting script:

    cuda_graphs, batch_size, topk_size, k, dtype, n_outer, n_inner, n_warmup,
    n_inner_inputs, method, args, compile, duration (seconds, one per outer
    step, each covering n_inner calls), device

Timing follows the reference's method (:98-146): optional capture of the
``n_inner`` calls in a CUDA graph, warm-up, then ``n_outer`` replays timed with
CUDA events, the inputs refilled with fresh normal samples before every step
(outside the timed region) and a device-side sleep queued in front of each
timed step so that the launches are already queued when the timer starts.

The default grid is the reference's (:264-327) without its RAFT rows (cupy and
pylibraft are not part of this build) and without ``torch.compile``: the
operator is a native custom op and is timed as such (``compile: null``).

    python benchmarks/measure_speed.py --out results/measure_speed.jsonl
    python benchmarks/measure_speed.py --quick            # a two-minute subset
"""

from __future__ import annotations

import argparse
import itertools
import json
import sys
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Iterable, Optional

import torch
from torch import Tensor

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from approx_topk import priority_queue  # noqa: E402
from approx_topk.experimental import bucketed_argmax  # noqa: E402

DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def torch_topk(xs: Tensor, k: int, dim: int) -> tuple[Tensor, Tensor]:
    return torch.topk(xs, k, dim, sorted=False)


METHOD_NAMES = {
    torch_topk: "__main__.torch_topk",
    priority_queue.topk: "approx_topk.priority_queue.topk",
    bucketed_argmax.topk_torch: "approx_topk.experimental.bucketed_argmax.topk_torch",
}


@dataclass(frozen=True)
class Experiment:
    method: Callable[..., tuple[Tensor, Tensor]]
    args: dict[str, Any]
    batch_size: int
    topk_size: int
    k: int
    dtype: torch.dtype
    cuda_graphs: bool
    n_outer: int
    n_inner: int
    n_warmup: int = 16
    n_inner_inputs: Optional[int] = None
    compile: Optional[str] = field(default=None)

    def record(self) -> dict[str, Any]:
        """The descriptive part of the output line (everything but the timings)."""
        return dict(
            cuda_graphs=self.cuda_graphs, batch_size=self.batch_size, topk_size=self.topk_size, k=self.k,
            n_outer=self.n_outer, n_inner=self.n_inner, n_warmup=self.n_warmup,
            n_inner_inputs=self.n_inner_inputs, args=dict(self.args), compile=self.compile,
            method=METHOD_NAMES[self.method], dtype=str(self.dtype).replace("torch.", ""),
        )

    def run(self) -> list[float]:
        n_inputs = self.n_inner if self.n_inner_inputs is None else self.n_inner_inputs
        if n_inputs > self.n_inner:
            raise ValueError("n_inner_inputs must not exceed n_inner")
        xs = torch.zeros(n_inputs, self.batch_size, self.topk_size, dtype=self.dtype, device="cuda")

        def inner() -> list[Tensor]:
            return [self.method(xs[i % n_inputs], k=self.k, dim=1, **self.args)[0] for i in range(self.n_inner)]

        return time_steps(inner, steps=self.n_outer, refill=lambda: torch.nn.init.normal_(xs),
                          cuda_graphs=self.cuda_graphs, warmup_steps=self.n_warmup)


def time_steps(fn: Callable[[], Any], steps: int, refill: Callable[[], Any] = lambda: None,
               cuda_graphs: bool = True, warmup_steps: Optional[int] = None) -> list[float]:
    """Seconds per step for ``steps`` steps of ``fn`` (CUDA events; ``refill`` runs
    before every step, outside the timed region)."""
    if cuda_graphs:
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):       # first call outside capture: lazy initialisation
            refill()
            fn()
        torch.cuda.current_stream().wait_stream(side)
        refill()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        fn = graph.replay
    for _ in range(steps if warmup_steps is None else warmup_steps):
        refill()
        fn()
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for start, end in events:
        refill()
        torch.cuda._sleep(10_000_000)       # keeps the GPU busy while the step's launches queue up
        start.record()
        fn()
        end.record()
    events[-1][1].synchronize()
    return [start.elapsed_time(end) / 1e3 for start, end in events]


def default_grid(ns: Iterable[int], batch_sizes: Iterable[int], dtype: torch.dtype,
                 graph_configs: list[dict[str, Any]]) -> list[Experiment]:
    """The reference's grid: n in ``ns``, k in {64, n/8}, exact top-k, the operator
    with j in {1, 2, 4} and both values of ``multithread_buckets``, and the k_b = 1
    arg-max entry."""
    out: list[Experiment] = []
    for n, batch, gc in itertools.product(ns, batch_sizes, graph_configs):
        for k in (64, n // 8):
            if k >= n:
                continue
            rows: list[tuple[Callable, dict[str, Any]]] = [(torch_topk, {})]
            for mtb in (False, True):
                for j in (1, 2, 4):
                    rows.append((priority_queue.topk, dict(j=j, k_mult=1, multithread_buckets=mtb)))
            rows.append((bucketed_argmax.topk_torch, dict(interleaved=True)))
            for method, args in rows:
                out.append(Experiment(method=method, args=args, batch_size=batch, topk_size=n, k=k,
                                      dtype=dtype, **gc))
    return out


def sweep(experiments: Iterable[Experiment], out: Path) -> None:
    out.parent.mkdir(parents=True, exist_ok=True)
    experiments = list(experiments)
    with out.open("w") as f:
        for idx, e in enumerate(experiments):
            rec = e.record()
            print(f"[{idx + 1}/{len(experiments)}] " + " ".join(f"{k}={v}" for k, v in rec.items()),
                  file=sys.stderr, flush=True)
            rec["duration"] = e.run()
            rec["device"] = torch.cuda.get_device_name()
            print(json.dumps(rec), file=f, flush=True)


def main(argv: Optional[list[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", type=Path, default=Path("results/measure_speed.jsonl"))
    ap.add_argument("--ns", type=int, nargs="+", default=[2**e for e in (16, 15, 14, 13, 12)])
    ap.add_argument("--batch-sizes", type=int, nargs="+", default=[128, 32])
    ap.add_argument("--dtype", choices=sorted(DTYPES), default="float32")
    ap.add_argument("--quick", action="store_true", help="two sizes, one batch size, short loops")
    args = ap.parse_args(argv)
    graph_configs = [dict(cuda_graphs=False, n_outer=512, n_inner=1),
                     dict(cuda_graphs=True, n_outer=16, n_inner=128)]
    ns, batches = args.ns, args.batch_sizes
    if args.quick:
        ns, batches = [2**16, 2**12], [128]
        graph_configs = [dict(cuda_graphs=False, n_outer=32, n_inner=1, n_warmup=4),
                         dict(cuda_graphs=True, n_outer=4, n_inner=16, n_warmup=2)]
    sweep(default_grid(ns, batches, DTYPES[args.dtype], graph_configs), args.out)
    print(f"wrote {args.out}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
