"""Read bandwidth per configuration from sweep logs of ``measure_speed.py``.

Accepts any number of JSONL files in the record layout of the reference's sweep
(this build's logs and the reference's own, e.g. its published H100 logs), so
that both can be put side by side.  The bandwidth is the reference's definition
(reference benchmarks/plot_bandwidth.py:41-47): bytes of input read per call,
``sizeof(dtype) * topk_size * batch_size``, over the mean time per call.
Prints a table (one line per configuration, one column per input file) instead
of a figure; ``--csv`` writes the same rows to a file.

    python benchmarks/bandwidth_table.py results/measure_speed.jsonl [other.jsonl ...]
"""

from __future__ import annotations

import argparse
import json
import re
import sys
from pathlib import Path

import numpy as np

ELEM_BYTES = {"float32": 4, "float16": 2, "bfloat16": 2, "float64": 8}


def short_name(method: str, args: dict) -> str:
    """`approx_topk.priority_queue.topk` + {j: 2} -> `priority_queue(j=2)`."""
    m = re.sub(r"\b(experimental|approx_topk|topk|__main__)\b", "", method)
    m = re.sub(r"\.+", ".", m).strip(".")
    a = ", ".join(f"{k}={v}" for k, v in args.items())
    return f"{m}({a})".replace("()", "") or "topk"


def load(path: Path) -> dict[tuple, dict]:
    rows = {}
    with path.open() as f:
        for line in f:
            if not line.strip():
                continue
            r = json.loads(line)
            per_call = float(np.mean(r["duration"])) / r["n_inner"]
            stderr = float(np.std(r["duration"]) / np.sqrt(len(r["duration"]))) / r["n_inner"]
            key = (r["dtype"], r["batch_size"], r["topk_size"], r["k"], bool(r["cuda_graphs"]),
                   r.get("compile") or "eager", short_name(r["method"], r.get("args") or {}))
            rows[key] = dict(seconds=per_call, stderr=stderr,
                             bandwidth=ELEM_BYTES[r["dtype"]] * r["topk_size"] * r["batch_size"] / per_call,
                             device=r.get("device", "?"))
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("logs", type=Path, nargs="+")
    ap.add_argument("--csv", type=Path)
    args = ap.parse_args(argv)
    tables = [load(p) for p in args.logs]
    keys = sorted(set().union(*[t.keys() for t in tables]))
    head = ["dtype", "batch", "n", "k", "graphs", "compile", "method"]
    cols = [f"{p.stem} GB/s" for p in args.logs]
    lines = [head + cols]
    for key in keys:
        cells = [f"{t[key]['bandwidth'] / 1e9:.1f}" if key in t else "-" for t in tables]
        lines.append([str(v) for v in key] + cells)
    widths = [max(len(row[i]) for row in lines) for i in range(len(lines[0]))]
    for row in lines:
        print("  ".join(c.ljust(w) for c, w in zip(row, widths)))
    for p, t in zip(args.logs, tables):
        devices = sorted({v["device"] for v in t.values()})
        print(f"# {p}: {len(t)} configurations, device(s): {', '.join(devices)}", file=sys.stderr)
    if args.csv:
        args.csv.parent.mkdir(parents=True, exist_ok=True)
        with args.csv.open("w") as f:
            for row in lines:
                f.write(",".join(c.replace(",", ";") for c in row) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
