"""The benchmark tools that mirror the reference's ``benchmarks/`` folder:
record layout and table arithmetic on the CPU, a miniature sweep and the recall
experiments on the GPU."""

import importlib.util
import json
import sys
from pathlib import Path

import pytest
import torch

BENCH = Path(__file__).resolve().parents[1] / "pytorch-approx-topk_b200" / "benchmarks"


def load(name):
    if str(BENCH) not in sys.path:
        sys.path.insert(0, str(BENCH))
    spec = importlib.util.spec_from_file_location(f"atk_bench_{name}", BENCH / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod          # dataclasses look their module up by name
    spec.loader.exec_module(mod)
    return mod


# fields of one line of the reference's sweep log (benchmarks/measure_speed.py:27-41, :244-250)
REFERENCE_FIELDS = {"cuda_graphs", "batch_size", "topk_size", "k", "dtype", "n_outer", "n_inner", "n_warmup",
                    "n_inner_inputs", "method", "args", "compile", "duration", "device"}


def test_sweep_record_layout():
    ms = load("measure_speed")
    grid = ms.default_grid([4096], [8], torch.float32, [dict(cuda_graphs=False, n_outer=2, n_inner=1)])
    # per (n, batch, graph mode): k in {64, n/8} x (exact + 3 j x 2 modes + arg-max)
    assert len(grid) == 2 * (1 + 6 + 1)
    rec = grid[1].record()
    assert set(rec) | {"duration", "device"} == REFERENCE_FIELDS
    assert rec["method"] == "approx_topk.priority_queue.topk" and rec["dtype"] == "float32"
    assert rec["args"] == dict(j=1, k_mult=1, multithread_buckets=False)
    json.dumps(rec)
    assert {e.record()["method"] for e in grid} == {
        "__main__.torch_topk", "approx_topk.priority_queue.topk",
        "approx_topk.experimental.bucketed_argmax.topk_torch"}


def test_bandwidth_table_arithmetic(tmp_path, capsys):
    bt = load("bandwidth_table")
    line = dict(cuda_graphs=True, batch_size=128, topk_size=65536, k=64, dtype="float32", n_outer=2, n_inner=4,
                n_warmup=1, n_inner_inputs=None, method="approx_topk.priority_queue.topk",
                args=dict(j=2, k_mult=1, multithread_buckets=False), compile=None,
                duration=[4e-5, 4e-5], device="test")
    log = tmp_path / "a.jsonl"
    log.write_text(json.dumps(line) + "\n")
    rows = bt.load(log)
    (key, row), = rows.items()
    assert key[-1] == "priority_queue(j=2, k_mult=1, multithread_buckets=False)"
    assert row["seconds"] == pytest.approx(1e-5)
    assert row["bandwidth"] == pytest.approx(4 * 65536 * 128 / 1e-5)
    assert bt.main([str(log), "--csv", str(tmp_path / "t.csv")]) == 0
    assert "3355.4" in capsys.readouterr().out
    assert (tmp_path / "t.csv").read_text().count("\n") == 2
    assert bt.short_name("__main__.torch_topk", {}) == "torch_topk"


def test_recall_helpers():
    rr = load("run_recall")
    ks = rr.valid_ks(128)
    assert ks[0] == 1024 and ks[-1] < rr.N and all(k % 4 == 0 for k in ks)
    rc = load("run_cumulative_recall")
    assert rc.first_below([1.0, 1.0, 0.95, 0.4], 0.99) == 3
    assert rc.first_below([1.0, 1.0], 0.5) == 3


@pytest.mark.gpu
def test_miniature_sweep_runs(tmp_path):
    ms = load("measure_speed")
    grid = ms.default_grid([4096], [8], torch.float32,
                           [dict(cuda_graphs=False, n_outer=3, n_inner=1, n_warmup=1),
                            dict(cuda_graphs=True, n_outer=2, n_inner=4, n_warmup=1)])
    out = tmp_path / "r" / "speed.jsonl"
    ms.sweep(grid, out)
    lines = [json.loads(l) for l in out.read_text().splitlines()]
    assert len(lines) == len(grid)
    for rec in lines:
        assert set(rec) == REFERENCE_FIELDS
        assert len(rec["duration"]) == rec["n_outer"] and all(0 < d < 1 for d in rec["duration"])
    bt = load("bandwidth_table")
    assert len(bt.load(out)) == len(grid)


@pytest.mark.gpu
def test_recall_experiments():
    rr = load("run_recall")
    rc = load("run_cumulative_recall")
    gen = torch.Generator(device="cuda").manual_seed(0)
    draw = rr.distributions(gen)["uniform"]
    m = rr.methods()
    k = rr.N // 8
    assert rr.recall_pair(draw(), m["exact"], k) == (1.0, 1.0)
    prev = 0.0
    for name in ("1 per bucket", "2 per bucket", "4 per bucket"):
        top_50, top_k = rr.recall_pair(draw(), m[name], k)
        assert 0.6 < top_k <= 1.0 and top_50 >= top_k - 0.05
        assert top_k > prev            # more survivors per bucket, higher recall
        prev = top_k
    curve = rc.cumulative_recall(draw(), m["exact"], k)
    assert len(curve) == k and min(curve) == 1.0
    curve = rc.cumulative_recall(draw(), m["4 per bucket"], k)
    assert curve[0] > 0.9 and curve[-1] < curve[0]
