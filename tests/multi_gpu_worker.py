"""Worker of tests/test_multi_gpu.py: one rank per GPU under torchrun (NCCL).

Checks on real GPUs that (1) the bucket-group sharding of one long row with either
exchange of the candidates (NCCL all-gather; stores into the peers' buffers over
NVLink) gives bit-identical results to the single-GPU operator on the same row, on
every rank, and (2) row sharding reproduces the unsharded result row for row.
"""

import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
for p in (str(ROOT), str(ROOT / "pytorch-approx-topk_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch
import torch.distributed as dist

import approx_topk
from approx_topk import distributed as atd


def trace(*what):
    if os.environ.get("ATK_WORKER_TRACE"):
        print(f"[rank {os.environ.get('RANK')}]", *what, file=sys.stderr, flush=True)


def canonical(v, i):
    o = torch.argsort(i)
    return v[o], i[o]


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    try:
        for dtype, n, k, j, k_mult in [(torch.float32, 1 << 22, 1 << 12, 4, 2), (torch.bfloat16, 1 << 20, 1 << 10, 2, 1),
                                       (torch.float16, 1 << 21, 1 << 16, 1, 2)]:
            g = torch.Generator(device=dev).manual_seed(4321)        # same row on every rank
            row = torch.randn(n, device=dev, generator=g).to(dtype)
            b = k * k_mult // j
            slab = atd.slab_of_row(row, b, rank, world)
            trace("long row", dtype, n, k, j, k_mult)
            v, i = atd.topk_long_row(slab, k, j, k_mult)
            trace("single-GPU operator")
            ev, ei = approx_topk.topk(row.view(1, -1), k, -1, j=j, k_mult=k_mult)
            (v, i), (ev, ei) = canonical(v, i), canonical(ev.view(-1), ei.view(-1))
            assert torch.equal(i, ei), f"rank {rank}: indices differ ({dtype}, n={n})"
            assert torch.equal(v.view(torch.int16 if v.element_size() == 2 else torch.int32),
                               ev.view(torch.int16 if ev.element_size() == 2 else torch.int32)), \
                f"rank {rank}: values differ ({dtype}, n={n})"
        # a bucket count the world size does not divide (padded last group), and the plan
        # with preallocated buffers, stepped directly and as a CUDA graph holding the collective
        for dtype, stripes, k, j, k_mult in [(torch.float32, 4096, 45, 3, 1), (torch.float16, 2048, 4099, 2, 2),
                                             (torch.float32, 1024, 1 << 15, 4, 2)]:
            b = k * k_mult // j
            g = torch.Generator(device=dev).manual_seed(777)
            row = torch.randn(stripes * b, device=dev, generator=g).to(dtype)
            slab = atd.slab_of_row(row, b, rank, world)
            ev, ei = approx_topk.topk(row.view(1, -1), k, -1, j=j, k_mult=k_mult)
            ev, ei = canonical(ev.view(-1), ei.view(-1))
            v, i = canonical(*atd.topk_long_row(slab, k, j, k_mult))
            assert torch.equal(i, ei) and torch.equal(v, ev), f"rank {rank}: padded groups differ ({dtype}, b={b})"
            # both exchanges: the NCCL all-gather, and the push over peer memory (two buffer
            # sets that alternate: a replayed graph holds an even number of steps)
            for exchange, graph_steps in (("all_gather", 1), ("push", 2)):
                trace("plan", exchange, dtype, stripes, k, j, k_mult)
                plan = atd.LongRowTopK(stripes, k, j, k_mult, dtype, dev, exchange=exchange)
                for _ in range(3):
                    v, i = canonical(*plan(slab))
                    assert torch.equal(i, ei) and torch.equal(v, ev), \
                        f"rank {rank}: plan differs ({exchange}, {dtype}, b={b})"
                torch.cuda.synchronize(dev)
                dist.barrier()
                trace("graph", exchange)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                    for _ in range(graph_steps):
                        plan(slab)
                plan.values.zero_()
                for _ in range(3):
                    graph.replay()
                torch.cuda.synchronize(dev)
                v, i = canonical(plan.values.clone(), plan.indices.clone())
                assert torch.equal(i, ei) and torch.equal(v, ev), \
                    f"rank {rank}: graph replay differs ({exchange}, {dtype}, b={b})"
                # a graph that holds a collective must be gone before the process group is torn down
                del graph
                torch.cuda.synchronize(dev)
                plan.close()
                dist.barrier()
                del plan
        # rows: each rank computes its span; together they equal the full batch
        g = torch.Generator(device=dev).manual_seed(99)
        x = torch.randn(37, 1 << 14, device=dev, generator=g)
        full_v, full_i = approx_topk.topk(x, 256, -1, j=2)
        lo, hi = atd.row_shard(x.shape[0], rank, world)
        v, i = atd.topk_row_sharded(x[lo:hi], 256, j=2)
        assert torch.equal(v, full_v[lo:hi]) and torch.equal(i, full_i[lo:hi])
        torch.cuda.synchronize(dev)
        dist.barrier()
        if rank == 0:
            print("MULTI_GPU_OK", world, flush=True)
    finally:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
