"""GPU tests of the k_b = 1 entry points (the cases of the reference's
tests/test_bucket_argmax.py: golden values in bucket order, transposed input,
and agreement between the entry points on random inputs)."""

from functools import partial

import numpy as np
import pytest
import torch

from approx_topk.experimental.bucketed_argmax import topk_torch, topk_triton
from oracle import cpu_oracle as oracle

pytestmark = pytest.mark.gpu

ENTRY_POINTS = [
    topk_torch,
    partial(topk_triton, block_size=1, kernel="bk"),
    partial(topk_triton, block_size=8, kernel="bk"),
    partial(topk_triton, block_size=1, kernel="bkn"),
    partial(topk_triton, block_size=8, kernel="bkn"),
]


@pytest.mark.parametrize("topk", ENTRY_POINTS)
def test_golden_values(topk):
    inputs = torch.stack([100 * torch.arange(0, 20), -100 * torch.arange(0, 20)]).to(
        dtype=torch.float32, device="cuda")
    values, indices = topk(inputs, k=3, dim=1, interleaved=False)
    assert torch.equal(values.cpu(), torch.tensor([[600.0, 1300, 1900], [0, -700, -1400]]))
    assert torch.equal(indices.cpu(), torch.tensor([[6, 13, 19], [0, 7, 14]]))

    values_t, indices_t = topk(inputs.T, k=3, dim=0, interleaved=False)
    assert torch.equal(values_t.T, values)
    assert torch.equal(indices_t.T, indices)

    values_i, indices_i = topk(inputs, k=3, dim=1, interleaved=True)
    assert torch.equal(values_i.cpu(), torch.tensor([[1800.0, 1900, 1700], [0, -100, -200]]))
    assert torch.equal(indices_i.cpu(), torch.tensor([[18, 19, 17], [0, 1, 2]]))


@pytest.mark.parametrize("interleaved", [False, True])
def test_fuzz_against_oracle(interleaved):
    # Random b, n, k as in the reference's fuzz (values are small integers, so
    # ties are frequent); integer inputs are cast to float32, which is exact.
    for seed in np.random.SeedSequence(123).generate_state(20):
        rng = np.random.RandomState(seed)
        torch.manual_seed(rng.randint(100000))
        b = 2 ** rng.randint(1, 5) if rng.rand() < 0.5 else rng.randint(1, 17)
        n = 2 ** rng.randint(1, 11) if rng.rand() < 0.5 else rng.randint(1, 1025)
        k = -(-n // rng.randint(1, 33))
        x = torch.randint(-(2 ** 15), 2 ** 15, (b, n), device="cuda").float()
        values, indices = topk_torch(x, k=k, dim=1, interleaved=interleaved)
        ov, oi = oracle.bucketed_argmax(x.cpu(), k, interleaved)
        assert torch.equal(values.cpu(), ov), (b, n, k)
        assert torch.equal(indices.cpu(), oi), (b, n, k)


def test_fixture_from_reference_topk_torch(golden):
    data, meta = golden
    dtypes = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}
    seen = 0
    for idx, m in enumerate(meta):
        if m["kind"] != "topk_torch":
            continue
        seen += 1
        x = torch.from_numpy(data[f"c{idx}_x"]).to(dtypes[m["dtype"]]).cuda()
        v, i = topk_torch(x, k=m["k"], dim=-1, interleaved=m["interleaved"])
        assert torch.equal(v.float().cpu(), torch.from_numpy(data[f"c{idx}_values"])), m
        if m["dtype"] == "float32":
            assert torch.equal(i.cpu(), torch.from_numpy(data[f"c{idx}_indices"])), m
    assert seen >= 10


def test_config_c1_shape_recall():
    # the reference's CPU-runnable configuration: fp32 16 x 65536, k = 256, interleaved
    g = torch.Generator().manual_seed(0)
    x = torch.randn(16, 65536, generator=g)
    v, i = topk_torch(x.cuda(), k=256, dim=-1, interleaved=True)
    ov, oi = oracle.bucketed_argmax(x, 256, True)
    assert torch.equal(v.cpu(), ov) and torch.equal(i.cpu(), oi)
    r = oracle.recall(x, v.cpu())
    assert 0.55 < r < 0.72      # analytic value for k_b = 1, b = k is about 0.63


def test_integer_input_first_maximum_wins():
    # ten distinct values over 64 positions: every bucket has tied maxima
    x = torch.randint(0, 10, (2, 64), device="cuda")
    v, i = topk_torch(x, k=4, dim=1, interleaved=True)
    ov, oi = oracle.bucketed_argmax(x.cpu(), 4, True)
    assert v.dtype == torch.int64
    assert torch.equal(v.cpu(), ov) and torch.equal(i.cpu(), oi)
