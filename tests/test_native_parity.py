"""GPU parity tests proper: the CUDA kernels, called through the C ABI, against
the CPU oracle (bit-exact values and indices, slot by slot) and, when it has
been built, against the reference's own CUDA operator."""

import pytest
import torch

from oracle import cpu_oracle as oracle
from tests import native_api as api
from tests import reference_cuda as refcuda
from tests.helper_funcs import assert_pairs_identical, assert_valid_selection

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16, torch.float16]


def make(rows, n, dtype, seed, dist="randn"):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dist == "randn":
        x = torch.randn(rows, n, generator=g, device="cuda")
    elif dist == "ties":       # few distinct values: ties at every bucket boundary
        x = torch.randint(-3, 4, (rows, n), generator=g, device="cuda").float()
    elif dist == "linspace":   # correlated rows
        x = torch.linspace(0, 1, n, device="cuda")[None] + 0.01 * torch.randn(rows, n, generator=g, device="cuda")
    else:
        raise ValueError(dist)
    return x.to(dtype)


def bits(t):
    t = t.detach().cpu()
    return t.view(torch.int32) if t.dtype == torch.float32 else t.view(torch.int16)


def check_stage1_exact(x, k0, j, interleaved):
    v, i = api.stage1(x, k0, j, interleaved)
    ov, oi = oracle.stage1(x.cpu(), k0, j, interleaved)
    assert torch.equal(bits(v), bits(ov)), f"values differ ({tuple(x.shape)}, k0={k0}, j={j}, il={interleaved})"
    assert torch.equal(i.cpu(), oi), f"indices differ ({tuple(x.shape)}, k0={k0}, j={j}, il={interleaved})"
    return v, i


# (rows, n, k0) geometries: aligned/unaligned, b | n and b !| n, tiny rows,
# few-row long-column shapes that take the split-and-merge path.
GEOMETRIES = [
    (4, 1024, 256), (3, 1001, 48), (5, 17, 8), (2, 1000, 500), (2, 4096, 4096),
    (7, 8192, 64), (1, 65536, 64), (2, 100000, 1024), (1, 12, 12), (33, 515, 24),
    # long columns (head-test kernel variant): unsplit aligned / unaligned, and split
    (2, 300000, 1024), (2, 300001, 1020), (1, 600000, 96), (3, 2 * 5000 * 300, 2 * 5000),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("j", [1, 2, 3, 4])
@pytest.mark.parametrize("interleaved", [True, False])
def test_stage1_matches_oracle_slot_for_slot(dtype, j, interleaved):
    for seed, (rows, n, k0) in enumerate(GEOMETRIES):
        if k0 % j:
            k0 = (k0 // j) * j
        if k0 == 0:
            continue
        check_stage1_exact(make(rows, n, dtype, 10 + seed), k0, j, interleaved)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("j", [1, 2, 4])
@pytest.mark.parametrize("interleaved", [True, False])
def test_stage1_tie_rule(dtype, j, interleaved):
    # Later position wins among equal values, exactly like the reference scan.
    for seed, (rows, n, k0) in enumerate([(4, 1024, 128), (2, 777, 28), (1, 65536, 32), (3, 30000, 512)]):
        check_stage1_exact(make(rows, n, dtype, 50 + seed, "ties"), k0, j, interleaved)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("j", [1, 2, 4])
def test_stage1_sixteen_bit_stripe_numbers_at_the_limit(dtype, j):
    # The packed queues of the 16-bit types hold the stripe number in 16 bits:
    # exactly 65536 stripes (with and without a ragged last one) still fit, one
    # more does not and takes the wide queues.  Tie-heavy data makes the last
    # stripes win, so a wrapped stripe number would show.
    b = 8
    for n in (65536 * b, 65536 * b - 3, 65536 * b + 3):
        for dist in ("ties", "randn"):
            check_stage1_exact(make(3, n, dtype, 60 + j, dist), b * j, j, True)
    # many rows: no stripe split inside the block, every thread walks all 65536 stripes
    check_stage1_exact(make(300, 65536 * 4, dtype, 61, "ties"), 4 * j, j, True)


def test_stage1_all_equal_row():
    x = torch.ones(2, 4096, device="cuda")
    v, i = check_stage1_exact(x, 64, 2, True)
    # 32 buckets of 128: the two last positions of every bucket survive
    assert i[0, :4].tolist() == [32 * 126, 32 * 127, 32 * 126 + 1, 32 * 127 + 1]


def test_stage1_neg_inf_is_selectable():
    x = torch.full((2, 256), float("-inf"), device="cuda")
    x[0, 5] = 1.0
    v, i = check_stage1_exact(x, 16, 2, True)
    assert (i >= 0).all() and (i < 256).all()


@pytest.mark.parametrize("dtype", DTYPES)
def test_stage1_long_columns_head_test_path(dtype):
    # l_full / splits >= 256 selects the variant that tests queue heads first.
    for j in (1, 2, 4):
        check_stage1_exact(make(64, 1 << 18, dtype, 7), 64 * j, j, True)
    check_stage1_exact(make(1, 1 << 20, dtype, 8, "ties"), 8, 4, True)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("j", [1, 2, 3, 4])
def test_stage1_stripes_split_over_blocks(dtype, j):
    # Few rows and few buckets: with scratch the stripes of a column are split over
    # several blocks and merged; the result must not depend on the scratch.
    lib = api._native.lib()
    for seed, (rows, n, k0) in enumerate([(1, 1 << 20, 64), (1, (1 << 20) + 77, 32), (2, 300000, 96),
                                          (3, 1 << 18, 16), (1, 1 << 22, 1024), (5, 1000003, 8)]):
        k0 = (k0 // j) * j
        assert lib.atk_stage1_workspace_bytes(api._native.dtype_code(dtype), rows, n, k0, j, 1) > 0
        for dist in ("randn", "ties"):
            x = make(rows, n, dtype, 950 + seed, dist)
            v, i = api.stage1(x, k0, j, True, use_workspace=True)
            v0, i0 = api.stage1(x, k0, j, True, use_workspace=False)
            assert torch.equal(bits(v), bits(v0)) and torch.equal(i, i0), (rows, n, k0, dist)
            ov, oi = oracle.stage1(x.cpu(), k0, j, True)
            assert torch.equal(bits(v), bits(ov)) and torch.equal(i.cpu(), oi), (rows, n, k0, dist)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32, torch.int16, torch.int8])
@pytest.mark.parametrize("j", [1, 2, 3, 4])
def test_stripe_split_with_a_short_remainder_has_no_made_up_candidates(dtype, j):
    # Stripe counts that leave the last block of a split fewer stripes than a queue
    # has entries (16385 = 128 * 128 + 1, 129 * 127 + 2, ...) on rows whose values
    # are all negative (log-probabilities): a never-filled queue slot written to a
    # scratch plane would outrank every real element.  b = 17 is not a multiple of
    # the vector width, so 16-bit rows take the scalar packed path.
    for b, stripes in [(17, 16385), (17, 129 * 127 + 2), (24, 16386), (8, 40001), (17, 16384 + 3)]:
        n = b * stripes
        k0 = b * j
        g = torch.Generator(device="cuda").manual_seed(b + stripes + j)
        if dtype.is_floating_point:
            x = (-torch.rand(1, n, device="cuda", generator=g) - 0.5).to(dtype)
        else:
            info = torch.iinfo(dtype)
            x = torch.randint(info.min, min(-1, info.min // 2 + 2), (1, n), device="cuda", generator=g).to(dtype)
        ov, oi = oracle.stage1(x.cpu(), k0, j, True)
        for use_workspace in (True, False):
            v, i = api.stage1(x, k0, j, True, use_workspace=use_workspace)
            assert torch.equal(v.cpu(), ov) and torch.equal(i.cpu(), oi), (dtype, b, stripes, j, use_workspace)
        if j == 4:                          # through the operator, which always passes the workspace
            from approx_topk import topk

            tv, ti = topk(x, k0, -1, j=j)
            assert torch.equal(tv.cpu(), ov) and torch.equal(ti.cpu(), oi)


def test_operator_single_row_small_k_uses_the_split_and_matches_oracle():
    from approx_topk import topk
    from approx_topk.experimental.bucketed_argmax import topk_torch

    x = make(1, 128256, torch.float16, 960)
    for j, k_mult in [(1, 1), (2, 1), (1, 4), (2, 4)]:
        v, i = topk(x, 64, -1, j=j, k_mult=k_mult)
        ov, oi = oracle.topk(x.cpu(), 64, j=j, k_mult=k_mult)
        assert_valid_selection(x, v, i, ov)
    v, i = topk_torch(x, 64, -1, True)
    ov, oi = oracle.bucketed_argmax(x.cpu(), 64, True)
    assert torch.equal(bits(v), bits(ov)) and torch.equal(i.cpu(), oi)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("j", [1, 2, 4])
def test_stage1_contiguous_bucket_lengths(dtype, j):
    # contiguous buckets from a few elements (shared-memory tile kernel) over
    # hundreds (lane groups, vector loads) to hundreds of thousands (block per
    # bucket), with row bases that are not 16-byte aligned
    for seed, (rows, n, k0) in enumerate([(3, 4096, 1024), (2, 4099, 400), (5, 9000, 96), (4, 128256, 256),
                                          (1, 1 << 20, 64), (2, 300000, 8), (1, (1 << 20) + 13, 28),
                                          (2, 50001, 12500)]):
        k0 = (k0 // j) * j
        for dist in ("randn", "ties"):
            base = make(rows, n + 3, dtype, 700 + seed, dist)
            x = base[:, 3:]                      # element-aligned only
            v, i = api.stage1(x, k0, j, False)
            ov, oi = oracle.stage1(x.cpu().contiguous(), k0, j, False)
            assert torch.equal(bits(v), bits(ov)), (rows, n, k0, dist)
            assert torch.equal(i.cpu(), oi), (rows, n, k0, dist)


def test_stage1_row_stride_and_unaligned_base():
    base = make(9, 1100, torch.float32, 3)
    view = base[:, 3:1027]            # base pointer only 4-byte aligned, row stride 1100
    v, i = api.stage1(view, 128, 2, True)
    ov, oi = oracle.stage1(view.cpu().contiguous(), 128, 2, True)
    assert torch.equal(bits(v), bits(ov)) and torch.equal(i.cpu(), oi)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("j", [1, 2, 3, 4])
@pytest.mark.parametrize("interleaved", [True, False])
def test_stage1_matches_reference_cuda_operator(dtype, j, interleaved):
    refcuda.require()
    for seed, (rows, n, k0) in enumerate(GEOMETRIES):
        k0 = (k0 // j) * j
        if k0 == 0:
            continue
        for dist in ("randn", "ties"):
            x = make(rows, n, dtype, 90 + seed, dist)
            v, i = api.stage1(x, k0, j, interleaved)
            rv, ri = refcuda.reference_stage1(x, k0, j, interleaved, multithread_buckets=False)
            # same slots, same order: the thread-per-bucket kernel's layout is kept
            assert torch.equal(bits(v), bits(rv)), (dtype, j, interleaved, rows, n, k0, dist)
            assert torch.equal(i, ri), (dtype, j, interleaved, rows, n, k0, dist)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("j,k_mult", [(1, 1), (2, 1), (4, 2), (2, 4), (1, 4)])
def test_topk_matches_reference_cuda_operator(dtype, j, k_mult):
    refcuda.require()
    for seed, (rows, n, k) in enumerate([(8, 4096, 64), (3, 10007, 32), (2, 65536, 1024)]):
        x = make(rows, n, dtype, 200 + seed)
        v, i = api.topk(x, k, j, k_mult, True)
        rv, ri = refcuda.reference_topk(x, k, -1, j, k_mult, True, False)
        if dtype == torch.float32:
            assert_pairs_identical(v, i, rv, ri)       # tie-free rows: bit-exact pairs
        else:
            assert_valid_selection(x, v, i, rv)        # ties: multiset + valid distinct indices
        assert oracle.recall(x.cpu(), v.cpu()) == oracle.recall(x.cpu(), rv.cpu())


@pytest.mark.parametrize("j", [1, 2, 4])
def test_block_per_bucket_reference_kernel_same_selection(j):
    refcuda.require()
    # The reference's 64-thread-per-bucket kernel must select the same set on tie-free rows.
    x = make(4, 16384, torch.float32, 77)
    v, i = api.stage1(x, 32 * j, j, True)
    rv, ri = refcuda.reference_stage1(x, 32 * j, j, True, multithread_buckets=True)
    assert_pairs_identical(v, i, rv, ri)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,k0,k", [(4, 256, 64), (16, 4096, 2048), (3, 1000, 1), (2, 1000, 1000),
                                       (5, 777, 300), (2, 16384, 5000), (2, 32768, 5000), (1, 40000, 20000),
                                       (2, 100000, 777), (1, 1 << 21, 1 << 20),
                                       (3, 20001, 5000), (2, 70003, 35001), (7, 4097, 100)])   # rows off the vector alignment
def test_select_matches_oracle(dtype, rows, k0, k):
    for dist in ("randn", "ties"):
        cv = make(rows, k0, dtype, 300 + k, dist)
        cv = torch.where(cv == 0, torch.zeros_like(cv), cv)      # no negative zeros
        ci = torch.randperm(rows * k0, device="cuda", generator=torch.Generator(device="cuda").manual_seed(k)
                            ).reshape(rows, k0)
        v, i = api.select(cv, ci, k)
        ov, oi = oracle.select(cv.cpu(), ci.cpu(), k)
        # lowest candidate slots win ties in both: identical pairs
        assert_pairs_identical(v, i, ov, oi)
        v2, i2 = api.select(cv, ci, k)
        assert torch.equal(v, v2) and torch.equal(i, i2)         # deterministic, order included


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64])
@pytest.mark.parametrize("rows,k0,k", [(80, 32768, 9000),       # 1280 chunks: more than one cooperative launch holds
                                       (160, 65536, 30000)])    # 5120 chunks: the count pass instead of the chained scan
def test_select_with_a_launch_per_pass_matches_oracle(dtype, rows, k0, k):
    """Problems too large for the one-launch select take the digit passes as separate
    launches (chained write pass for few chunks, a count pass for many)."""
    for dist in ("randn", "ties"):
        cv = make(rows, k0, dtype, 900 + k, dist)
        cv = torch.where(cv == 0, torch.zeros_like(cv), cv)
        ci = torch.randperm(rows * k0, device="cuda", generator=torch.Generator(device="cuda").manual_seed(k)
                            ).reshape(rows, k0)
        v, i = api.select(cv, ci, k)
        ov, oi = oracle.select(cv.cpu(), ci.cpu(), k)
        assert_pairs_identical(v, i, ov, oi)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.int16, torch.int8, torch.float32])
def test_two_stage_odd_candidate_counts_and_views(dtype):
    # Candidate counts that are not multiples of the vector width, j = 3, a
    # strided input view: the 8/16-bit types take the packed hand-off between the
    # stages (entries instead of values + positions), fp32 the plain one.
    def data(rows, n, seed):
        g = torch.Generator(device="cuda").manual_seed(seed)
        if dtype.is_floating_point:
            return torch.randn(rows, n, generator=g, device="cuda").to(dtype)
        info = torch.iinfo(dtype)
        return torch.randint(info.min, info.max + 1, (rows, n), generator=g, device="cuda").to(dtype)

    for seed, (rows, n, k, j, k_mult) in enumerate([(5, 1000, 9, 3, 2), (3, 777, 5, 1, 3), (2, 4099, 14, 2, 5),
                                                    (4, 50000, 1023, 1, 3), (1, 300, 21, 3, 4)]):
        x = data(rows, n, 700 + seed)
        v, i = api.topk(x, k, j, k_mult, True)
        ov, oi = oracle.topk(x.cpu(), k, j, k_mult, True)
        assert_valid_selection(x, v, i, ov)
        if dtype == torch.float32:
            assert_pairs_identical(v, i, ov, oi)
    base = data(6, 2100, 710)
    view = base[:, 50:2050]                      # row stride 2100, 100-byte offset
    v, i = api.topk(view, 64, 2, 2, True)
    ov, oi = oracle.topk(view.cpu().contiguous(), 64, 2, 2, True)
    assert_valid_selection(view, v, i, ov)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("j,k_mult", [(1, 2), (2, 2), (4, 2), (2, 4), (1, 16)])
def test_topk_two_stage_matches_oracle(dtype, j, k_mult):
    for seed, (rows, n, k) in enumerate([(8, 4096, 64), (3, 10007, 32), (2, 65536, 1024), (1, 300000, 20000)]):
        if k * k_mult > n:
            continue
        x = make(rows, n, dtype, 400 + seed)
        v, i = api.topk(x, k, j, k_mult, True)
        ov, oi = oracle.topk(x.cpu(), k, j, k_mult, True)
        assert_valid_selection(x, v, i, ov)
        if dtype == torch.float32:
            assert_pairs_identical(v, i, ov, oi)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("j,k_mult", [(1, 2), (2, 2), (3, 2), (4, 2), (2, 4), (1, 4)])
def test_two_stage_many_rows_matches_oracle_and_two_kernel_path(dtype, j, k_mult):
    # Many rows, so that stage 1 runs unsplit and (for 16-bit elements) hands packed
    # entries to the select: aligned, ragged (b does not divide n), unaligned rows, long
    # columns, and the largest candidate count it takes.
    for seed, (rows, n, k) in enumerate([(96, 4096, 96), (80, 10007, 48), (77, 8190, 24), (100, 131072, 12),
                                         (75, 65536, 2040)]):
        k = (k // j) * j if (k * k_mult) % j else k
        if (k * k_mult) % j:
            continue
        for dist in ("randn", "ties"):
            x = make(rows, n, dtype, 800 + seed, dist)
            v, i = api.topk(x, k, j, k_mult, True)
            ov, oi = oracle.topk(x.cpu(), k, j, k_mult, True)
            assert_valid_selection(x, v, i, ov)
            if dtype == torch.float32 and dist == "randn":
                assert_pairs_identical(v, i, ov, oi)
            # the operator and stage 1 + select called separately agree bit for bit (same tie choices)
            cv, ci = api.stage1(x, k * k_mult, j, True)
            sv, si = api.select(cv, ci, k)
            if not (dtype != torch.float32 and dist == "ties"):
                assert torch.equal(bits(v), bits(sv)) and torch.equal(i, si), (rows, n, k, dist)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("interleaved", [True, False])
def test_bucketed_argmax_matches_oracle(dtype, interleaved):
    for seed, (rows, n, k) in enumerate([(2, 20, 3), (3, 1000, 7), (4, 4096, 256), (2, 10, 4), (1, 5, 8),
                                         (16, 65536, 256), (2, 1001, 64), (2, 300000, 64), (2, 300001, 63),
                                         (2, 400000, 1024), (1, 400003, 1021)]):
        for dist in ("randn", "ties"):
            x = make(rows, n, dtype, 500 + seed, dist)
            v, i = api.bucketed_argmax(x, k, interleaved)
            ov, oi = oracle.bucketed_argmax(x.cpu(), k, interleaved)
            assert torch.equal(bits(v), bits(ov)), (rows, n, k, dist)
            assert torch.equal(i.cpu(), oi), (rows, n, k, dist)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("j", [1, 4])
def test_slab_gives_the_matching_slice_of_the_full_row(dtype, j):
    stripes, b, groups = 512, 2048, 4
    x = make(1, stripes * b, dtype, 600)
    full_v, full_i = api.stage1(x, b * j, j, True)
    cols = b // groups
    for g in range(groups):
        slab = x.view(stripes, b)[:, g * cols:(g + 1) * cols].contiguous()
        v, i = api.stage1_slab(slab, b, g * cols, j)
        assert torch.equal(bits(v), bits(full_v[0, g * cols * j:(g + 1) * cols * j]))
        assert torch.equal(i, full_i[0, g * cols * j:(g + 1) * cols * j])


@pytest.mark.parametrize("dtype,j,k_mult", [(torch.float32, 2, 1), (torch.bfloat16, 4, 2)])
def test_host_buffer_entry_point_equals_device_path(dtype, j, k_mult):
    x = make(37, 8192, dtype, 700)
    v, i = api.topk(x, 128, j, k_mult, True)
    hv, hi = api.topk_host(x.cpu().pin_memory(), 128, j, k_mult, True, chunk_rows=5)
    assert torch.equal(bits(hv), bits(v)) and torch.equal(hi, i.cpu())
    hv, hi = api.topk_host(x.cpu(), 128, j, k_mult, True)      # pageable memory, default chunking
    assert torch.equal(bits(hv), bits(v)) and torch.equal(hi, i.cpu())


def test_long_row_entry_point_single_rank_equals_operator():
    # world size 1: the bucket-group path (slab stage 1 + select) must equal the plain operator
    from approx_topk import distributed as atd

    n, k, j, k_mult = 1 << 20, 1 << 12, 4, 2
    row = make(1, n, torch.float32, 900)
    slab = atd.slab_of_row(row.view(-1), k * k_mult // j, 0, 1)
    v, i = atd.topk_long_row(slab, k, j, k_mult)
    ev, ei = api.topk(row, k, j, k_mult, True)
    assert_pairs_identical(v.view(1, -1), i.view(1, -1), ev, ei)


def test_long_row_plan_with_preallocated_buffers_and_strided_slab():
    # LongRowTopK (buffers allocated once, graph-capturable step) equals topk_long_row, step after
    # step; a strided column range passed as the slab is copied, not read through its base pointer
    from approx_topk import distributed as atd

    n, k, j, k_mult = 1 << 21, 1 << 14, 4, 2      # 2^15 candidates: the multi-block select with its workspace
    b = k * k_mult // j
    row = make(1, n, torch.float32, 901)
    plan = atd.LongRowTopK(n // b, k, j, k_mult, torch.float32, row.device)
    ev, ei = api.topk(row, k, j, k_mult, True)
    for _ in range(2):
        v, i = plan(row.view(n // b, b))
        assert_pairs_identical(v.view(1, -1), i.view(1, -1), ev, ei)
    # a strided slab: columns [64, 192) of the view as one "rank" of a wider row
    view = row.view(n // b, b)[:, 64:192]
    assert not view.is_contiguous()
    sv, si = atd._native_stage1_slab(view, b, 64, j)
    dv, di = api.stage1_slab(view.contiguous(), b, 64, j)
    assert torch.equal(bits(sv), bits(dv)) and torch.equal(si, di)
    # CUDA-graph capture of a step (what the benchmark times)
    g = torch.cuda.CUDAGraph()
    slab = row.view(n // b, b)
    torch.cuda.synchronize()
    with torch.cuda.graph(g):
        plan(slab)
    plan.values.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert_pairs_identical(plan.values.view(1, -1), plan.indices.view(1, -1), ev, ei)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("j", [2, 3, 4])
def test_stage1_short_columns_two_pass_scan(dtype, j):
    # 16-bit floats, an even number of buckets and fewer than 256 stripes per thread take the
    # two-pass scan (threshold from a values-only network, then only the elements at or above it
    # enter the exact queues): every chunk length (16 / 32 / 64 stripes, several chunks, short last
    # chunks), a ragged last stripe, stripes split inside the block, tie-heavy rows, rows full of
    # one value and rows holding -inf must all agree with the serial scan slot for slot.
    shapes = []
    for stripes in (j, 5, 15, 16, 17, 31, 32, 33, 63, 64, 65, 100, 128, 129, 200, 255):
        if stripes < j:
            continue
        for b, rem, rows in ((2, 0, 3), (6, 3, 5), (64, 0, 40), (1026, 17, 2), (4096, 0, 9)):
            shapes.append((rows, stripes * b + rem, b * j))
    # enough 256-column tiles to occupy the GPU: the shared-memory tile kernel, one chunk, several
    # chunks (later chunks use the queues' weakest entries as the threshold), a short last chunk, a
    # ragged last stripe, a partial last tile
    for rows, b, stripes, rem in ((450, 256, 64, 0), (450, 256, 300, 17), (230, 512, 1100, 0), (120, 1000, 65, 999),
                                  (500, 264, 16, 0), (460, 256, 33, 5)):
        shapes.append((rows, stripes * b + rem, b * j))
    for seed, (rows, n, k0) in enumerate(shapes):
        for dist in ("randn", "ties"):
            check_stage1_exact(make(rows, n, dtype, 3000 + seed, dist), k0, j, True)
    x = make(4, 64 * 130, dtype, 1)
    x[0] = 1.5                                    # one value everywhere: the latest stripes win
    x[1, ::3] = float("-inf")
    x[2] = float("-inf")
    x[2, 77] = 0.25
    x[3, : 64 * 100] = -0.0                       # both zeros tie; the sign of the input is returned
    x[3, 64 * 100:] = 0.0
    check_stage1_exact(x, 64 * j, j, True)
    x = make(460, 256 * 130, dtype, 2)            # the same special rows through the tile kernel
    x[0] = 1.5
    x[1, ::3] = float("-inf")
    x[2] = float("-inf")
    x[2, 77] = 0.25
    x[3, : 256 * 100] = -0.0
    x[3, 256 * 100:] = 0.0
    x[4, 5::7] = float("nan")                     # NaNs are outside the contract; nothing may crash or hang
    v, i = api.stage1(x, 256 * j, j, True)
    ov, oi = oracle.stage1(x[:4].cpu(), 256 * j, j, True)
    assert torch.equal(bits(v[:4]), bits(ov)) and torch.equal(i[:4].cpu(), oi)
    assert bool(((i[4] >= 0) & (i[4] < x.shape[1])).all())
    # the packed hand-off to the select on such shapes (k_mult > 1)
    for rows, n, k, k_mult in ((70, 65536, 512 * j, 2), (33, 12 * 1000 + 5, 6 * j, 2), (300, 4096, 32 * j, 4),
                               (500, 65536, 512 * j, 2), (450, 256 * 70 + 3, 64 * j, 4)):
        for dist in ("randn", "ties"):
            xx = make(rows, n, dtype, 3100 + rows, dist)
            v, i = api.topk(xx, k, j, k_mult, True)
            ov, oi = oracle.topk(xx.cpu(), k, j, k_mult, True)
            assert_valid_selection(xx, v, i, ov)


@pytest.mark.parametrize("j", [2, 3, 4])
def test_stage1_float32_long_columns_tile_kernel(j):
    # float32 columns of 1024 stripes or more with enough 128-column tiles take the shared-memory
    # tile kernel: one split, stripes split over blocks (with scratch) and not (without), a ragged
    # last stripe, a partial last tile, several chunks with a short last one, ties, -inf.
    # (queues of three or four entries take it from 64 stripes on)
    for seed, (rows, b, stripes, rem) in enumerate(((4, 4096, 1500, 77), (1, 8192, 2049, 0), (30, 512, 1100, 3),
                                                    (500, 128, 1024, 0), (7, 1000, 1030, 999), (2, 16384, 1024, 5),
                                                    (40, 2048, 64, 0), (9, 8192, 100, 4097), (600, 128, 70, 1),
                                                    (40, 2048, 600, 8))):
        n, k0 = stripes * b + rem, b * j
        for dist in ("randn", "ties"):
            x = make(rows, n, torch.float32, 4000 + seed, dist)
            if dist == "randn":
                x[0, ::5] = float("-inf")
            ov, oi = oracle.stage1(x.cpu(), k0, j, True)
            for use_workspace in (True, False):
                v, i = api.stage1(x, k0, j, True, use_workspace=use_workspace)
                assert torch.equal(bits(v), bits(ov)) and torch.equal(i.cpu(), oi), (rows, b, stripes, rem, dist, use_workspace)
    # through the operator (second stage behind it) and the slab entry point of the long-row path
    x = make(2, 2048 * 4096, torch.float32, 4100)
    v, i = api.topk(x, 2048 * j, j, 2, True)
    ov, oi = oracle.topk(x.cpu(), 2048 * j, j, 2, True)
    assert_pairs_identical(v, i, ov, oi)
    slab = x[0].view(2048, 4096)[:, 1024:3072].contiguous()
    sv, si = api.stage1_slab(slab, 4096, 1024, j)
    fv, fi = api.stage1(x[:1], 4096 * j, j, True)
    assert torch.equal(bits(sv), bits(fv[0, 1024 * j:3072 * j])) and torch.equal(si, fi[0, 1024 * j:3072 * j])
