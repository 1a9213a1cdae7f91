"""GPU parity for the element types beyond fp32 / bf16 / fp16: float64, int64,
int32, int16, int8 and uint8 -- the rest of the reference's native dispatch
(approx_topk/priority_queue_approx_topk.cu:449-453).  The CUDA kernels, called
through the C ABI and through the Python operator, against the CPU oracle (slot
for slot), the reference's CPU outputs (committed fixtures) and, when it has
been built, the reference's own CUDA operator."""

import numpy as np
import pytest
import torch

from approx_topk import topk
from approx_topk.experimental.bucketed_argmax import topk_torch, topk_triton
from oracle import cpu_oracle as oracle
from tests import native_api as api
from tests import reference_cuda as refcuda
from tests.helper_funcs import assert_pairs_identical, assert_valid_selection

pytestmark = pytest.mark.gpu

WIDE = [torch.float64, torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8]
NAMES = {str(t).replace("torch.", ""): t for t in WIDE}


def make(rows, n, dtype, seed, dist="full"):
    """full: the whole value range with the extreme values planted;
    ties: seven distinct values, so every bucket boundary is a tie."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dist == "ties":
        x = torch.randint(0, 7, (rows, n), generator=g, device="cuda")
        return x.to(dtype) if dtype == torch.uint8 else (x - 3).to(dtype)
    if dtype == torch.float64:
        x = torch.randn(rows, n, generator=g, device="cuda", dtype=torch.float64) * 1e100
        if n > 8:
            x[:, 5] = float("-inf")
            x[:, n - 2] = float("inf")
        return x
    info = torch.iinfo(dtype)
    if dtype == torch.int64:
        hi = torch.randint(-2**31, 2**31, (rows, n), generator=g, device="cuda")
        lo = torch.randint(0, 2**32, (rows, n), generator=g, device="cuda")
        x = hi * 2**32 + lo
    else:
        x = torch.randint(info.min, info.max + 1, (rows, n), generator=g, device="cuda").to(dtype)
    if n > 8:
        x[:, 3] = info.min
        x[:, n // 2] = info.max
        x[:, n - 1] = info.min
    return x


def check_stage1_exact(x, k0, j, interleaved):
    v, i = api.stage1(x, k0, j, interleaved)
    ov, oi = oracle.stage1(x.cpu(), k0, j, interleaved)
    tag = f"({x.dtype}, {tuple(x.shape)}, k0={k0}, j={j}, il={interleaved})"
    assert v.dtype == x.dtype
    if x.dtype == torch.float64:
        assert torch.equal(v.cpu().view(torch.int64), ov.view(torch.int64)), "values differ " + tag
    else:
        assert torch.equal(v.cpu(), ov), "values differ " + tag
    assert torch.equal(i.cpu(), oi), "indices differ " + tag


# (rows, n, k0): aligned / unaligned bucket counts, ragged last stripe, tiny
# rows, few-row long-column shapes (in-block and cross-block stripe splits,
# head-test variant), short and long contiguous buckets.
GEOMETRIES = [
    (4, 1024, 256), (3, 1001, 48), (5, 17, 8), (2, 1000, 500), (2, 4096, 4096),
    (7, 8192, 64), (1, 65536, 64), (2, 100000, 1024), (1, 12, 12), (33, 515, 24),
    (2, 300001, 1020), (1, 600000, 96), (1, 400000, 12),
]


@pytest.mark.parametrize("dtype", WIDE)
@pytest.mark.parametrize("j", [1, 2, 3, 4])
@pytest.mark.parametrize("interleaved", [True, False])
def test_stage1_matches_oracle_slot_for_slot(dtype, j, interleaved):
    for seed, (rows, n, k0) in enumerate(GEOMETRIES):
        k0 = (k0 // j) * j
        for dist in ("full", "ties"):
            check_stage1_exact(make(rows, n, dtype, 10 * seed + j, dist), k0, j, interleaved)


@pytest.mark.parametrize("dtype", WIDE)
@pytest.mark.parametrize("interleaved", [True, False])
def test_rows_full_of_the_lowest_value(dtype, interleaved):
    # Every bucket holds exactly j elements, all equal to the type's lowest value
    # (the value the queues start from): every position must come back once.
    low = float("-inf") if dtype.is_floating_point else torch.iinfo(dtype).min
    for j in (1, 2, 4):
        x = torch.full((3, 64), low, device="cuda", dtype=dtype)
        check_stage1_exact(x, 64, j, interleaved)
        v, i = api.stage1(x, 64, j, interleaved)
        assert torch.equal(i.sort(dim=-1).values.cpu(), torch.arange(64).expand(3, 64))
        assert bool((v == low).all())
        # longer buckets: the last j positions of every bucket win
        x = torch.full((2, 640), low, device="cuda", dtype=dtype)
        check_stage1_exact(x, 64, j, interleaved)


@pytest.mark.parametrize("dtype", WIDE)
def test_stage1_without_scratch_and_on_views(dtype):
    # no workspace: the split over blocks is off, same answer
    x = make(1, 600000, dtype, 5)
    v, i = api.stage1(x, 96, 2, True, use_workspace=False)
    ov, oi = oracle.stage1(x.cpu(), 96, 2, True)
    assert torch.equal(v.cpu(), ov) and torch.equal(i.cpu(), oi)
    # a view whose base pointer and row stride break the vector alignment
    base = make(9, 1100, dtype, 6)
    view = base[:, 3:1027]
    v, i = api.stage1(view, 128, 2, True)
    ov, oi = oracle.stage1(view.cpu().contiguous(), 128, 2, True)
    assert torch.equal(v.cpu(), ov) and torch.equal(i.cpu(), oi)


@pytest.mark.parametrize("dtype", WIDE)
@pytest.mark.parametrize("rows,k0,k", [
    (5, 256, 64), (3, 4096, 2048), (2, 16384, 5000), (2, 8192, 8191),   # one block per row
    (2, 20000, 777), (1, 300000, 150000), (3, 70000, 1),                # several blocks per row
    (3, 20001, 5000), (2, 70003, 35001),                                # ... with rows that break the vector alignment
])
def test_select_matches_oracle(dtype, rows, k0, k):
    for dist in ("full", "ties"):
        cv = make(rows, k0, dtype, k0 + k, dist)
        ci = torch.randperm(rows * k0, device="cuda").reshape(rows, k0)
        v, i = api.select(cv, ci, k)
        ov, oi = oracle.select(cv.cpu(), ci.cpu(), k)
        # same winners, ties at the boundary resolved towards the lowest slot in both
        assert_pairs_identical(v, i, ov, oi)


@pytest.mark.parametrize("dtype", WIDE)
@pytest.mark.parametrize("j,k_mult", [(1, 1), (2, 1), (4, 2), (2, 4), (3, 2)])
def test_topk_matches_oracle(dtype, j, k_mult):
    for seed, (rows, n, k) in enumerate([(8, 4096, 12 * j), (3, 10007, 6 * j), (2, 65536, 1020 // j * j)]):
        for dist in ("full", "ties"):
            x = make(rows, n, dtype, 100 + seed, dist)
            v, i = api.topk(x, k, j, k_mult, True)
            ov, oi = oracle.topk(x.cpu(), k, j, k_mult, True)
            assert_pairs_identical(v, i, ov, oi)


def test_reference_cpu_fixtures(golden_all_dtypes):
    data, meta = golden_all_dtypes
    seen = 0
    for idx, m in enumerate(meta):
        x = torch.from_numpy(data[f"c{idx}_x"]).cuda()
        ev = torch.from_numpy(data[f"c{idx}_values"])
        ei = torch.from_numpy(data[f"c{idx}_indices"])
        if m["kind"] == "bucketed_torch_topk":
            v, i = topk(x, m["k"], dim=-1, j=m["j"], k_mult=m["k_mult"], interleaved=m["interleaved"])
            assert v.dtype == x.dtype and i.dtype == torch.int64
            assert torch.equal(v.cpu().sort(dim=-1).values, ev), m
            assert torch.equal(x.gather(-1, i), v), m
            s = x.sort(dim=-1).values
            if not bool((s[:, 1:] == s[:, :-1]).any()):
                assert torch.equal(i.cpu().sort(dim=-1).values, ei), m
        else:
            v, i = topk_torch(x, k=m["k"], dim=-1, interleaved=m["interleaved"])
            assert torch.equal(v.cpu(), ev) and torch.equal(i.cpu(), ei), m
        seen += 1
    assert seen >= 90


def test_int64_arg_max_fuzz():
    # Random small shapes in the spirit of the reference's Triton fuzz test
    # (tests/test_bucket_argmax.py:76-110): int64 input from randint, contiguous
    # buckets, k = ceil(n / m) so that padding is exercised; both kernel names of
    # the reference's signature must agree with the CPU restatement exactly.
    rng = np.random.RandomState(321)
    for _ in range(40):
        rows = int(rng.randint(1, 17))
        n = int(2 ** rng.randint(1, 11)) if rng.rand() < 0.5 else int(rng.randint(1, 1025))
        k = -(-n // int(rng.randint(1, 33)))
        block_size = int(2 ** rng.randint(0, 5))
        x = torch.randint(-(2**15), 2**15, (rows, n), device="cuda")
        assert x.dtype == torch.int64
        for interleaved in (False, True):
            ov, oi = oracle.bucketed_argmax(x.cpu(), k, interleaved)
            for kernel in ("bk", "bkn"):
                v, i = topk_triton(x, k=k, dim=1, interleaved=interleaved, block_size=block_size, kernel=kernel)
                assert torch.equal(v.cpu(), ov) and torch.equal(i.cpu(), oi), (rows, n, k, interleaved)


@pytest.mark.parametrize("dtype", WIDE)
def test_operator_surface(dtype):
    x = make(6, 2048, dtype, 42)
    v, i = topk(x, 64, dim=-1, j=2, k_mult=2)
    ov, oi = oracle.topk(x.cpu(), 64, 2, 2, True)
    assert_pairs_identical(v, i, ov, oi)
    # single bucket along another dim (the only dim != last case the reference allows)
    y = make(30, 25 * 16, dtype, 43).reshape(30, 25, 16)
    v, i = topk(y, 3, dim=1, j=3)
    ev, _ = torch.topk(y.cpu(), 3, dim=1)
    assert torch.equal(v.cpu().sort(dim=1).values, ev.sort(dim=1).values)
    assert torch.equal(y.gather(1, i), v)
    torch.library.opcheck(topk, args=(x,), kwargs=dict(k=64, dim=-1, j=2, k_mult=2, interleaved=True))


def test_unsupported_dtype_is_rejected_clearly():
    x = torch.randn(2, 64, device="cuda") > 0
    with pytest.raises(RuntimeError, match="not supported"):
        topk(x, 4, dim=-1)
    with pytest.raises(RuntimeError, match="not supported"):
        topk_torch(x, k=4, dim=1, interleaved=True)


@pytest.mark.parametrize("dtype", WIDE)
@pytest.mark.parametrize("j", [1, 2, 3, 4])
@pytest.mark.parametrize("interleaved", [True, False])
def test_stage1_matches_reference_cuda_operator(dtype, j, interleaved):
    refcuda.require()
    for seed, (rows, n, k0) in enumerate(GEOMETRIES[:10]):
        k0 = (k0 // j) * j
        for dist in ("full", "ties"):
            x = make(rows, n, dtype, 90 + seed, dist)
            if dtype == torch.float64:
                x = x.clamp(min=-1e300)      # the reference never selects -inf (its sentinel is finite)
            v, i = api.stage1(x, k0, j, interleaved)
            rv, ri = refcuda.reference_stage1(x, k0, j, interleaved, multithread_buckets=False)
            # same slots, same order: the thread-per-bucket kernel's layout is kept
            assert torch.equal(v, rv), (dtype, j, interleaved, rows, n, k0, dist)
            assert torch.equal(i, ri), (dtype, j, interleaved, rows, n, k0, dist)


@pytest.mark.parametrize("dtype", WIDE)
@pytest.mark.parametrize("j,k_mult", [(2, 1), (4, 2), (1, 4)])
def test_topk_matches_reference_cuda_operator(dtype, j, k_mult):
    refcuda.require()
    for seed, (rows, n, k) in enumerate([(8, 4096, 64), (3, 10007, 32), (2, 65536, 1024)]):
        x = make(rows, n, dtype, 200 + seed)
        if dtype == torch.float64:
            x = x.clamp(min=-1e300)
        v, i = api.topk(x, k, j, k_mult, True)
        rv, ri = refcuda.reference_topk(x, k, -1, j, k_mult, True, False)
        assert_valid_selection(x, v, i, rv)
