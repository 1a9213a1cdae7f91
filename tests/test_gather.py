"""The record gather that follows the operator: against ``torch.gather`` on the
same indices (bit-exact, it only moves bytes)."""

import pytest
import torch

from approx_topk import topk
from approx_topk.gather import gather_records

pytestmark = pytest.mark.gpu


def reference(src, idx):
    return torch.gather(src, -2, idx.unsqueeze(-1).expand(*idx.shape, src.shape[-1]))


@pytest.mark.parametrize("dtype,d", [(torch.bfloat16, 128), (torch.float32, 64), (torch.float16, 100),
                                     (torch.float16, 7), (torch.uint8, 3), (torch.float64, 5), (torch.int32, 1)])
def test_matches_torch_gather(dtype, d):
    g = torch.Generator(device="cuda").manual_seed(d)
    src = (torch.randn(6, 4, 500, d, generator=g, device="cuda") * 50).to(dtype)
    idx = torch.randint(0, 500, (6, 4, 37), generator=g, device="cuda")
    out = gather_records(src, idx)
    assert out.shape == (6, 4, 37, d) and out.dtype == dtype
    assert torch.equal(out, reference(src, idx))


def test_keys_of_the_selected_positions():
    # attention-style use: scores [heads, seq], keys [heads, seq, d]
    g = torch.Generator(device="cuda").manual_seed(0)
    keys = torch.randn(16, 8192, 128, generator=g, device="cuda").bfloat16()
    q = torch.randn(16, 1, 128, generator=g, device="cuda").bfloat16()
    scores = (q @ keys.transpose(-1, -2)).squeeze(1)
    _, idx = topk(scores, 256, dim=-1, j=2, k_mult=2)
    out = gather_records(keys, idx)
    assert torch.equal(out, reference(keys, idx))


def test_views_single_row_and_empty():
    g = torch.Generator(device="cuda").manual_seed(1)
    big = torch.randn(3, 300, 40, generator=g, device="cuda")
    src = big[:, 10:210, :]                      # row stride larger than n*d, records still dense
    idx = torch.randint(0, 200, (3, 9), generator=g, device="cuda")
    assert torch.equal(gather_records(src, idx), reference(src, idx))
    one = torch.randn(77, 12, generator=g, device="cuda")
    i1 = torch.randint(0, 77, (5,), generator=g, device="cuda")
    assert torch.equal(gather_records(one, i1), one[i1])
    assert gather_records(one, i1[:0]).shape == (0, 12)
    narrow = big[:, :, :16]                      # records not dense: copied first
    assert torch.equal(gather_records(narrow, idx), reference(narrow, idx))


def test_out_of_range_positions_give_zero_records():
    src = torch.ones(2, 10, 4, device="cuda")
    idx = torch.tensor([[0, 10, 3], [-1, 9, 99]], device="cuda")
    out = gather_records(src, idx)
    assert out[0, 1].abs().sum() == 0 and out[1, 0].abs().sum() == 0 and out[1, 2].abs().sum() == 0
    assert out[0, 0].sum() == 4 and out[1, 1].sum() == 4


def test_argument_checks():
    src = torch.ones(2, 10, 4, device="cuda")
    with pytest.raises(ValueError):
        gather_records(src, torch.zeros(2, 3, device="cuda", dtype=torch.int32))
    with pytest.raises(ValueError):
        gather_records(src, torch.zeros(3, 3, device="cuda", dtype=torch.int64))
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        gather_records(src.cpu(), torch.zeros(2, 3, dtype=torch.int64))
