"""CPU (gloo, world_size 2) tests of the multi-GPU host logic: row sharding and
the bucket-group sharding of one long row with the all-gather of candidates.
The kernels are replaced by the CPU oracle so that only the partitioning, the
exchange and the index arithmetic are under test."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from approx_topk import distributed as atd
from oracle import cpu_oracle as oracle


def test_row_shard_covers_all_rows_once():
    for rows in (0, 1, 7, 128, 1000):
        for world in (1, 2, 3, 8):
            spans = [atd.row_shard(rows, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == rows
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        atd.row_shard(10, 2, 2)


def test_bucket_groups_pad_the_last_groups():
    assert atd.bucket_group(1024, 3, 4) == (768, 1024)
    # the world size does not divide the bucket count: full groups first, then short or empty ones
    assert [atd.bucket_group(10, r, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 9), (9, 10)]
    assert [atd.bucket_group(5, r, 4) for r in range(4)] == [(0, 2), (2, 4), (4, 5), (5, 5)]
    for b in (1, 5, 10, 17, 1024):
        for world in (1, 2, 3, 4, 8):
            spans = [atd.bucket_group(b, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == b
            assert all(x[1] == y[0] for x, y in zip(spans, spans[1:]))
            assert all(x[1] - x[0] <= atd.group_width(b, world) for x in spans)
    with pytest.raises(ValueError):
        atd.bucket_group(10, 4, 4)


def test_slab_cut_from_a_row_view_gives_the_dense_slabs_candidates():
    # a column range of the stripes x buckets view is strided; its candidates must be
    # those of the dense copy (the native entry point copies such a view before reading it,
    # which tests/test_native_parity.py checks on the GPU)
    row = torch.randn(64 * 16, generator=torch.Generator().manual_seed(3))
    view = row.view(64, 16)[:, 4:12]
    assert not view.is_contiguous()
    v, i = oracle_stage1_slab(view, 16, 4, 2)
    dv, di = oracle_stage1_slab(view.contiguous(), 16, 4, 2)
    assert torch.equal(v, dv) and torch.equal(i, di)
    assert torch.equal(row[i], v)


def oracle_stage1_slab(slab, total_buckets, col_offset, j):
    stripes, cols = slab.shape
    v, i = oracle.stage1(slab.reshape(1, -1), cols * j, j, interleaved=True)
    i = i.reshape(-1)
    return v.reshape(-1), (i // cols) * total_buckets + col_offset + (i % cols)


def oracle_select(cand_vals, cand_idx, k):
    v, i = oracle.select(cand_vals.reshape(1, -1), cand_idx.reshape(1, -1), k)
    return v.reshape(-1), i.reshape(-1)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, k, j, k_mult, n, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        row = torch.randn(n, generator=torch.Generator().manual_seed(1234))
        b = k * k_mult // j
        slab = atd.slab_of_row(row, b, rank, world)
        v, i = atd.topk_long_row(slab, k, j, k_mult, stage1=oracle_stage1_slab, select=oracle_select)
        torch.save((v, i), os.path.join(out, f"r{rank}.pt"))
        # rows: every rank handles its own span, nothing is exchanged
        start, stop = atd.row_shard(10, rank, world)
        torch.save((start, stop), os.path.join(out, f"span{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("k,j,k_mult,world,n", [(64, 2, 1, 2, 1 << 14), (64, 4, 2, 2, 1 << 14), (32, 1, 4, 2, 1 << 14),
                                                 (30, 2, 1, 2, 15 * 700),      # 15 buckets over 2 ranks: 8 + 7
                                                 (10, 2, 1, 3, 5 * 512),       # 5 buckets over 3 ranks: 2 + 2 + 1
                                                 (4, 2, 2, 3, 4 * 300)])       # 4 buckets over 3 ranks: 2 + 2 + 0
def test_long_row_ranks_equal_single_process(tmp_path, k, j, k_mult, world, n):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, k, j, k_mult, n, str(tmp_path)), nprocs=world, join=True)
    row = torch.randn(n, generator=torch.Generator().manual_seed(1234))
    ev, ei = oracle.topk(row.reshape(1, -1), k, j=j, k_mult=k_mult, interleaved=True)
    results = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    for v, i in results:
        assert torch.equal(v.sort().values, ev.reshape(-1).sort().values)
        assert torch.equal(i.sort().values, ei.reshape(-1).sort().values)
        assert torch.equal(row[i], v)
    for v, i in results[1:]:
        assert torch.equal(results[0][0], v) and torch.equal(results[0][1], i)
    spans = [torch.load(tmp_path / f"span{r}.pt") for r in range(world)]
    assert spans == [atd.row_shard(10, r, world) for r in range(world)]


def test_long_row_single_process_matches_oracle():
    n, k, j, k_mult = 1 << 13, 32, 2, 2
    row = torch.randn(n, generator=torch.Generator().manual_seed(7))
    slab = atd.slab_of_row(row, k * k_mult // j, 0, 1)
    v, i = atd.topk_long_row(slab, k, j, k_mult, stage1=oracle_stage1_slab, select=oracle_select)
    ev, ei = oracle.topk(row.reshape(1, -1), k, j=j, k_mult=k_mult)
    assert torch.equal(i.sort().values, ei.reshape(-1).sort().values)


def _failing_worker(rank, world, port, out):
    """Rank 1 fails on the host before the exchange; rank 0 must get an error from
    the collective (short process-group timeout), not hang."""
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=10))
    row = torch.randn(1 << 12, generator=torch.Generator().manual_seed(1))
    slab = atd.slab_of_row(row, 64, rank, world)
    if rank == 1:
        os._exit(17)                      # the rank disappears between steps, nothing in flight
    try:
        atd.topk_long_row(slab, 64, 1, 1, stage1=oracle_stage1_slab, select=oracle_select)
        outcome = "no error"
    except Exception as exc:              # noqa: BLE001 - any surfaced failure is the point
        outcome = f"error: {type(exc).__name__}"
    with open(os.path.join(out, "rank0.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)


def test_peer_failure_surfaces_as_an_error_not_a_hang(tmp_path):
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    assert all(not p.is_alive() for p in procs), "a rank hung after its peer failed"
    assert procs[1].exitcode == 17
    assert (tmp_path / "rank0.txt").read_text().startswith("error:")
