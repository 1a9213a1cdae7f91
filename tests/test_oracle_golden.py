"""Pins the CPU oracle (oracle/atk_oracle.c) to the reference.

(1) Every golden vector / known-answer case the reference's own tests hold for
    the path, restated here as data:
      tests/test_bucket_argmax.py:51-73   k_b = 1 goldens (values and indices, bucket order)
      tests/test_autobucket.py:88-127     arange cases
      tests/test_autobucket.py:23-51      ideally distributed top-k, contiguous, n = 1025
      tests/test_priority_queue.py:141-244 ideally distributed cases n = 17 / 10 000
      tests/test_priority_queue.py:71-138 bucket size one => exact
      tests/test_priority_queue.py:12-56  one bucket => exact
(2) Fixtures produced by importing the reference's Python modules
    (tests/golden/make_golden.py).
"""

import pytest
import torch

from oracle import cpu_oracle as oracle
from tests.helper_funcs import assert_close_up_to_permutation

DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def test_bucketed_argmax_known_answers():
    x = torch.stack([100 * torch.arange(0, 20), -100 * torch.arange(0, 20)]).float()
    v, i = oracle.bucketed_argmax(x, 3, interleaved=False)
    assert torch.equal(v, torch.tensor([[600.0, 1300, 1900], [0, -700, -1400]]))
    assert torch.equal(i, torch.tensor([[6, 13, 19], [0, 7, 14]]))
    v, i = oracle.bucketed_argmax(x, 3, interleaved=True)
    assert torch.equal(v, torch.tensor([[1800.0, 1900, 1700], [0, -100, -200]]))
    assert torch.equal(i, torch.tensor([[18, 19, 17], [0, 1, 2]]))


@pytest.mark.parametrize("interleaved,k_mult,k,expected", [
    (False, 1, 3, [3, 6, 9]),          # buckets {0..3} {4..6} {7..9}
    (True, 1, 3, [9, 7, 8]),           # buckets {0,3,6,9} {1,4,7} {2,5,8}
])
def test_arange_cases(interleaved, k_mult, k, expected):
    x = torch.arange(10).float()
    v, i = oracle.topk(x, k, j=1, k_mult=k_mult, interleaved=interleaved)
    assert_close_up_to_permutation(v, torch.tensor(expected).float())
    assert_close_up_to_permutation(i, torch.tensor(expected))


@pytest.mark.parametrize("interleaved,expected", [(False, [15, 13, 11, 9]), (True, [15, 14, 13, 12])])
def test_arange_k_mult_two(interleaved, expected):
    x = torch.arange(16).float()
    v, i = oracle.topk(x, 4, j=1, k_mult=2, interleaved=interleaved)
    assert_close_up_to_permutation(v, torch.tensor(expected).float())
    assert_close_up_to_permutation(i, torch.tensor(expected))


def _check_exact(x, k, j, interleaved, k_mult=1):
    v, i = oracle.topk(x, k, j=j, k_mult=k_mult, interleaved=interleaved)
    ev, ei = torch.topk(x, k, dim=-1)
    assert_close_up_to_permutation(v, ev)
    assert_close_up_to_permutation(i, ei)


def test_ideally_distributed_contiguous_1025():
    x = torch.zeros(2, 1025)
    for r, cols, vals in [
        (0, [1, 2, 300, 301, 600, 601, 900, 901], [10, 11, 11, 12, 11, 12, 13, 12]),
        (1, [5, 6, 302, 305, 610, 611, 920, 921], [10, 11, 11, 12, 11, 12, 13, 12]),
    ]:
        x[r, cols] = torch.tensor(vals).float()
    v, i = oracle.topk(x, 8, j=2, interleaved=False)
    ev, ei = torch.topk(x, 8, dim=-1)
    assert_close_up_to_permutation(v, ev)
    assert_close_up_to_permutation(i, ei)


def test_ideally_distributed_n17():
    # contiguous buckets [0..4] [5..8] [9..12] [13..16]
    x = torch.zeros(2, 17)
    x[0, [0, 4, 5, 8, 9, 12, 13, 16]] = torch.arange(11.0, 19.0)
    x[1, [2, 3, 6, 7, 10, 11, 14, 15]] = torch.arange(21.0, 29.0)
    _check_exact(x, 8, 2, interleaved=False)
    # interleaved buckets [0 4 8 12 16] [1 5 9 13] [2 6 10 14] [3 7 11 15]
    x = torch.zeros(2, 17)
    x[0, [0, 16, 1, 13, 2, 14, 3, 15]] = torch.arange(11.0, 19.0)
    x[1, [4, 8, 5, 9, 6, 10, 7, 11]] = torch.arange(21.0, 29.0)
    _check_exact(x, 8, 2, interleaved=True)


def test_ideally_distributed_long_sequence():
    # 4 contiguous buckets of 2500; spikes every 625 positions (4 per bucket),
    # two of each bucket's four made large so the exact top-8 has two per bucket.
    n, stride = 10_000, 625
    g = torch.Generator().manual_seed(1)
    x = torch.zeros(2, n)
    for r, first in ((0, 0), (1, 50)):
        pos = torch.arange(first, n, stride)
        vals = torch.rand(len(pos), generator=g) + 2.0
        vals[(torch.arange(len(pos)) % 4) < 2] += 1.0
        x[r, pos] = vals
    _check_exact(x, 8, 2, interleaved=False)


@pytest.mark.parametrize("interleaved", [False, True])
def test_bucket_size_one_is_exact(interleaved):
    g = torch.Generator().manual_seed(856)
    for n in (10, 16):
        _check_exact(torch.randn(n, generator=g), n, 1, interleaved)
    x = torch.randn(32, 1024, generator=g)
    _check_exact(x, 64, 1, interleaved, k_mult=16)


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("k", [2, 4])
def test_one_bucket_is_exact(interleaved, k):
    g = torch.Generator().manual_seed(234)
    _check_exact(torch.randn(1001, generator=g), k, k, interleaved)


def test_reference_fixtures(golden):
    data, meta = golden
    assert len(meta) >= 30
    for i, m in enumerate(meta):
        x = torch.from_numpy(data[f"c{i}_x"]).to(DTYPES[m["dtype"]])
        ev = torch.from_numpy(data[f"c{i}_values"])
        ei = torch.from_numpy(data[f"c{i}_indices"])
        if m["kind"] == "bucketed_torch_topk":
            v, idx = oracle.topk(x, m["k"], j=m["j"], k_mult=m["k_mult"], interleaved=m["interleaved"])
            assert torch.equal(v.float().sort(dim=-1).values, ev), m
            # 16-bit random rows contain ties, where the index choice is the
            # implementation's; fp32 rows are tie-free and pin the indices too.
            if m["dtype"] == "float32":
                assert torch.equal(idx.sort(dim=-1).values, ei), m
            else:
                assert torch.equal(x.float().gather(-1, idx), v.float()), m
        else:
            v, idx = oracle.bucketed_argmax(x, m["k"], interleaved=m["interleaved"])
            assert torch.equal(v.float(), ev), m
            if m["dtype"] == "float32":
                assert torch.equal(idx, ei), m


def _rows_have_ties(x):
    s = x.reshape(-1, x.shape[-1]).sort(dim=-1).values
    return bool((s[:, 1:] == s[:, :-1]).any())


def test_reference_fixtures_all_dtypes(golden_all_dtypes):
    # float64 and the integer element types of the reference's native dispatch,
    # against the reference's Python (CPU) path run on the same inputs.
    data, meta = golden_all_dtypes
    assert len(meta) >= 90
    seen = set()
    for i, m in enumerate(meta):
        x = torch.from_numpy(data[f"c{i}_x"])
        assert str(x.dtype) == "torch." + m["dtype"]
        seen.add(m["dtype"])
        ev = torch.from_numpy(data[f"c{i}_values"])
        ei = torch.from_numpy(data[f"c{i}_indices"])
        if m["kind"] == "bucketed_torch_topk":
            v, idx = oracle.topk(x, m["k"], j=m["j"], k_mult=m["k_mult"], interleaved=m["interleaved"])
            assert v.dtype == x.dtype
            assert torch.equal(v.sort(dim=-1).values, ev), m
            assert torch.equal(x.gather(-1, idx), v), m
            if not _rows_have_ties(x):        # tie-free rows pin the indices too
                assert torch.equal(idx.sort(dim=-1).values, ei), m
        else:
            v, idx = oracle.bucketed_argmax(x, m["k"], interleaved=m["interleaved"])
            assert torch.equal(v, ev), m
            assert torch.equal(idx, ei), m    # first maximum wins in both
    assert seen == {"float64", "int64", "int32", "int16", "int8", "uint8"}


def test_tie_rule_last_wins():
    # Reference insertion rule (priority_queue_approx_topk.cu:58-79): of equal
    # values the later position survives; slots ascend inside a bucket.
    x = torch.tensor([[1.0, 1.0, 1.0, 1.0, 1.0, 1.0]])
    v, i = oracle.stage1(x, 2, 2, interleaved=True)
    assert i.tolist() == [[4, 5]]
    v, i = oracle.stage1(x, 4, 2, interleaved=True)      # buckets {0,2,4} {1,3,5}
    assert i.tolist() == [[2, 4, 3, 5]]


def test_sentinel_modes():
    x = torch.tensor([[float("-inf"), 0.0, float("-inf"), float("-inf")]])
    v, i = oracle.stage1(x, 2, 2, interleaved=True, sentinel=oracle.lowest(torch.float32))
    assert i.tolist() == [[-1, 1]]                        # -inf never enters the reference queue
    v, i = oracle.stage1(x, 2, 2, interleaved=True)       # -inf start: every slot is a real element
    assert i.tolist() == [[3, 1]]


def test_timed_cpu_path_matches_reference_fixtures(golden, golden_all_dtypes):
    # oracle/torch_cpu_path.py is what bench.py times as the reference's CPU path
    # (the denominator of the speed-up); it must return what the reference's own
    # Python returned on the same inputs.
    from oracle.torch_cpu_path import bucketed_argmax_cpu, bucketed_topk_cpu

    checked = 0
    for (data, meta), widened in ((golden, True), (golden_all_dtypes, False)):
        for i, m in enumerate(meta):
            x = torch.from_numpy(data[f"c{i}_x"])
            if widened:
                x = x.to(DTYPES[m["dtype"]])
            ev = torch.from_numpy(data[f"c{i}_values"])
            ei = torch.from_numpy(data[f"c{i}_indices"])
            if m["kind"] == "bucketed_torch_topk":
                v, idx = bucketed_topk_cpu(x, m["k"], m["j"], m["k_mult"], m["interleaved"])
                got = v.float() if widened else v
                assert torch.equal(got.sort(dim=-1).values, ev), m
                # the reference pads with the type's lowest value; a row that holds that
                # value itself can have a padded position returned for it
                collides = not x.dtype.is_floating_point and bool((x == torch.iinfo(x.dtype).min).any())
                if not collides:
                    assert torch.equal(x.gather(-1, idx), v), m
                if not _rows_have_ties(x):
                    assert torch.equal(idx.sort(dim=-1).values, ei), m
            else:
                v, idx = bucketed_argmax_cpu(x, m["k"], m["interleaved"])
                assert torch.equal(v.float() if widened else v, ev), m
                if not _rows_have_ties(x):
                    assert torch.equal(idx, ei), m
            checked += 1
    assert checked >= 120
