"""The reference configurations at their FULL sizes on the GPU, checked (a)
directly against the reference's own CUDA operator on the same seeded input —
stage-1 candidates slot for slot, final (value, index) pairs bit-exact on
tie-free rows, the tie-tolerant rule otherwise, and the same recall — and (b)
through size-independent properties (the CPU oracle would take minutes there);
plus the reduced-size versions of the same recipes against the oracle and the
reference's CUDA operator, recall included.

Properties for stage 1 (k_mult = 1), bucket c = columns {c, c+b, ...}:
  * every returned index lies in its slot's bucket and points at its value;
  * slots of a bucket ascend; the last slot is the bucket maximum (torch.amax);
  * the multiset of the j values equals torch.topk of the bucket (exact per bucket).
For two-stage results: values are the k largest of the stage-1 candidates
(torch.topk), indices point at their values and are distinct.
"""

import pytest
import torch

from approx_topk import topk
from oracle import cpu_oracle as oracle
from tests import native_api as api
from tests import reference_cuda as refcuda
from tests.helper_funcs import assert_valid_selection

pytestmark = pytest.mark.gpu


def gen(kind, rows, n, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if kind == "randn":
        return torch.randn(rows, n, device="cuda", generator=g).to(dtype)
    if kind == "attention":
        x = torch.empty(rows, n, device="cuda", dtype=dtype)
        for r0 in range(0, rows, 32):
            nr = min(32, rows - r0)
            keys = torch.randn(nr, n, 128, device="cuda", generator=g)
            q = torch.randn(nr, 1, 128, device="cuda", generator=g)
            x[r0:r0 + nr] = (q @ keys.transpose(-1, -2) / 128 ** 0.5).squeeze(1).to(dtype)
        return x
    if kind == "spikes":
        x = torch.empty(rows, n, device="cuda", dtype=dtype)
        for r0 in range(0, rows, 256):
            nr = min(256, rows - r0)
            blk = 2.0 * torch.randn(nr, n, device="cuda", generator=g)
            pos = torch.rand(nr, n, device="cuda", generator=g).topk(16, dim=-1).indices
            blk.scatter_add_(1, pos, torch.full_like(pos, 8.0, dtype=blk.dtype))
            x[r0:r0 + nr] = blk.to(dtype)
        return x
    if kind == "linspace":
        return (torch.linspace(0, 1, n, device="cuda")[None]
                + 0.01 * torch.randn(rows, n, device="cuda", generator=g)).to(dtype)
    raise ValueError(kind)


def check_stage1_properties(x, v, i, j):
    rows, n = x.shape
    k0 = v.shape[-1]
    b = k0 // j
    assert n % b == 0
    slot_bucket = torch.arange(k0, device=x.device) // j
    assert torch.equal(i % b, slot_bucket.expand(rows, k0))
    assert torch.equal(x.gather(-1, i), v)
    vb = v.view(rows, b, j).float()
    assert bool((vb[..., 1:] >= vb[..., :-1]).all())
    buckets = x.view(rows, n // b, b)
    assert torch.equal(buckets.amax(dim=1), v.view(rows, b, j)[..., -1])
    for r0 in range(0, rows, 32):          # exact per-bucket top-j, in row blocks to bound memory
        blk = buckets[r0:r0 + 32].transpose(1, 2).float()
        want = blk.topk(j, dim=-1).values.flip(-1)
        assert torch.equal(want, vb[r0:r0 + 32])


def check_two_stage_properties(x, v, i, k, j, k_mult):
    rows = x.shape[0]
    cv, ci = api.stage1(x, k * k_mult, j, True)
    check_stage1_properties(x, cv, ci, j)
    want = cv.float().topk(k, dim=-1).values
    assert torch.equal(v.float().sort(dim=-1, descending=True).values, want)
    assert torch.equal(x.gather(-1, i), v)
    si = i.sort(dim=-1).values
    assert bool((si[:, 1:] != si[:, :-1]).all())


def bits_equal(a, b):
    """Bit-exact equality of two device tensors of the same element type."""
    view = {1: torch.int8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[a.element_size()]
    return a.dtype == b.dtype and torch.equal(a.view(view), b.view(view))


def recall_hits(x, v, k):
    """Per row: how many returned values reach the exact k-th largest (the
    numerator of the reference's recall, benchmarks/run_recall.py:27-36)."""
    hits = []
    for r0 in range(0, x.shape[0], 256):       # row blocks bound the float copy
        xf = x[r0:r0 + 256].float()
        kth = xf.topk(k, dim=-1).values[:, -1:]
        hits.append((v[r0:r0 + 256].float() >= kth).sum(dim=-1))
    return torch.cat(hits)


def assert_valid_selection_on_device(x, v, i, ref_v):
    """The tie-tolerant acceptance rule without leaving the GPU (rows too large
    to move): same value multiset as the reference, every index points at its
    value, indices distinct."""
    assert bits_equal(v.sort(dim=-1).values, ref_v.sort(dim=-1).values), "value multiset differs"
    assert bits_equal(x.gather(-1, i), v), "an index does not point at its value"
    si = i.sort(dim=-1).values
    assert bool((si[:, 1:] != si[:, :-1]).all()), "duplicate indices in a row"


def assert_same_pairs_on_device(v, i, ref_v, ref_i):
    """Identical (value, index) pairs per row, compared after sorting by index
    (indices are distinct, so that order is canonical)."""
    o, ro = i.argsort(dim=-1), ref_i.argsort(dim=-1)
    assert torch.equal(i.gather(-1, o), ref_i.gather(-1, ro)), "selected indices differ"
    assert bits_equal(v.gather(-1, o), ref_v.gather(-1, ro)), "selected values differ"


def test_c2_full_size_fp32_128x2p20_k65536_j2():
    x = gen("randn", 128, 1 << 20, torch.float32, 0)
    v, i = topk(x, 1 << 16, -1, j=2)
    check_stage1_properties(x, v, i, 2)
    # the reference's CUDA operator on the same rows: k_mult = 1 keeps its slot
    # layout, so values and indices agree slot for slot
    refcuda.require()
    rv, ri = refcuda.reference_topk(x, 1 << 16, -1, 2, 1, True, False)
    assert bits_equal(v, rv) and torch.equal(i, ri)
    assert torch.equal(recall_hits(x, v, 1 << 16), recall_hits(x, rv, 1 << 16))
    # recall equals the analytic value of the reference's model within sampling noise (0.7293)
    kth = x.topk(1 << 16, dim=-1).values[:, -1:]
    recall = (v >= kth).float().mean().item()
    assert abs(recall - 0.7293) < 0.01


def test_c3_full_size_bf16_1024x65536_k2048_j4_kmult2():
    x = gen("attention", 1024, 65536, torch.bfloat16, 1)
    v, i = topk(x, 2048, -1, j=4, k_mult=2)
    check_two_stage_properties(x, v, i, 2048, 4, 2)
    refcuda.require()
    # stage 1: the 4096 candidates of every row, slot for slot (bf16 rows are full of ties)
    cv, ci = api.stage1(x, 4096, 4, True)
    rcv, rci = refcuda.reference_stage1(x, 4096, 4, True, False)
    assert bits_equal(cv, rcv) and torch.equal(ci, rci)
    # whole operator: ties at the k-th value are torch.topk's choice in the reference
    rv, ri = refcuda.reference_topk(x, 2048, -1, 4, 2, True, False)
    assert_valid_selection_on_device(x, v, i, rv)
    assert torch.equal(recall_hits(x, v, 2048), recall_hits(x, rv, 2048))


@pytest.mark.parametrize("j", [1, 2])
@pytest.mark.parametrize("kind", ["spikes", "linspace"])
def test_c4_full_size_fp16_4096x128256_k64_kmult4(j, kind):
    x = gen(kind, 4096, 128256, torch.float16, 2)
    v, i = topk(x, 64, -1, j=j, k_mult=4)
    check_two_stage_properties(x, v, i, 64, j, 4)
    hits = recall_hits(x, v, 64)
    recall = hits.float().mean().item() / 64
    assert recall > (0.85 if j == 1 else 0.94)          # analytic: 0.886 / 0.969 for i.i.d. rows
    refcuda.require()
    cv, ci = api.stage1(x, 256, j, True)
    rcv, rci = refcuda.reference_stage1(x, 256, j, True, False)
    assert bits_equal(cv, rcv) and torch.equal(ci, rci)
    rv, ri = refcuda.reference_topk(x, 64, -1, j, 4, True, False)
    assert_valid_selection_on_device(x, v, i, rv)
    assert torch.equal(hits, recall_hits(x, rv, 64))     # recall equals the reference operator's, row by row


def test_c5b_slice_single_long_row():
    # the long-row recipe at 2^28 elements with the full configuration's bucket length (8192 stripes)
    n, k, j, k_mult = 1 << 28, 1 << 16, 4, 2
    x = gen("randn", 1, n, torch.float32, 3)
    v, i = topk(x, k, -1, j=j, k_mult=k_mult)
    check_two_stage_properties(x, v, i, k, j, k_mult)


def test_c5b_full_size_single_row_of_2p32():
    # The long row at its real size on one GPU (16 GiB of input): offsets beyond
    # 2^31 elements, 8192 stripes, 2^21 candidates, exact select down to 2^20.
    n, k, j, k_mult = 1 << 32, 1 << 20, 4, 2
    k0 = k * k_mult
    x = torch.empty(1, n, device="cuda", dtype=torch.float32)
    g = torch.Generator(device="cuda").manual_seed(5)
    for off in range(0, n, 1 << 28):
        x[0, off:off + (1 << 28)] = torch.randn(1 << 28, device="cuda", generator=g)
    refcuda.require()
    # stage 1 against the reference's kernel (grid of 16384 warps, 64-bit index math)
    cv, ci = api.stage1(x, k0, j, True)
    rcv, rci = refcuda.reference_stage1(x, k0, j, True, False)
    assert bits_equal(cv, rcv) and torch.equal(ci, rci)
    assert int(ci.max()) >= (1 << 31)                    # positions past the 32-bit range are reported
    del rcv, rci
    # the operator: same value multiset as the reference's torch.topk over the candidates
    v, i = topk(x, k, -1, j=j, k_mult=k_mult)
    want = cv.topk(k, dim=-1).values
    assert_valid_selection_on_device(x, v, i, want)
    # candidates above the k-th value are all selected; ties at it come from the candidates
    kth = want[:, -1:]
    sure = ci[cv > kth].sort().values
    got = i[v > kth].sort().values
    assert torch.equal(sure, got)
    # the bucket-group entry point on the whole row gives the same candidates
    sv, si = api.stage1_slab(x.view(n // (k0 // j), k0 // j), k0 // j, 0, j)
    assert bits_equal(sv.view(1, -1), cv) and torch.equal(si.view(1, -1), ci)


REDUCED = [
    # (name, kind, dtype, rows, n, k, j, k_mult)
    ("c1", "randn", torch.float32, 16, 65536, 256, 1, 1),
    ("c2", "randn", torch.float32, 4, 1 << 20, 1 << 16, 2, 1),
    ("c3", "attention", torch.bfloat16, 64, 65536, 2048, 4, 2),
    ("c4-spikes-j1", "spikes", torch.float16, 64, 128256, 64, 1, 4),
    ("c4-spikes-j2", "spikes", torch.float16, 64, 128256, 64, 2, 4),
    ("c4-corr-j1", "linspace", torch.float16, 64, 128256, 64, 1, 4),
    ("c4-corr-j2", "linspace", torch.float16, 64, 128256, 64, 2, 4),
    ("c5b-slice", "randn", torch.float32, 1, 1 << 24, 1 << 12, 4, 2),
]


@pytest.mark.parametrize("name,kind,dtype,rows,n,k,j,k_mult", REDUCED, ids=[r[0] for r in REDUCED])
def test_reduced_configs_match_oracle_and_reference_recall(name, kind, dtype, rows, n, k, j, k_mult):
    x = gen(kind, rows, n, dtype, 10)
    v, i = topk(x, k, -1, j=j, k_mult=k_mult)
    ov, oi = oracle.topk(x.cpu(), k, j=j, k_mult=k_mult)
    assert_valid_selection(x, v, i, ov)
    ours = oracle.recall(x.cpu(), v.cpu())
    assert ours == oracle.recall(x.cpu(), ov)
    refcuda.require()
    rv, ri = refcuda.reference_topk(x, k, -1, j, k_mult, True, False)
    assert_valid_selection(x, v, i, rv)
    assert ours == oracle.recall(x.cpu(), rv.cpu())       # recall equals the reference operator's
    if dtype == torch.float32:
        assert_same_pairs_on_device(v, i, rv, ri)
