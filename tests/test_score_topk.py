"""Fused score producer (atk_score_topk / approx_topk.attention.score_topk): the scores of
one query per row against the row's keys are computed inside the kernel and fed to the
bucketed top-k.

Two checks.  (1) Float work, tolerance: the scores (atk_scores writes them with the fused
kernel's arithmetic) agree with a double-precision reference within one unit in the last
place of the 16-bit result, and with the reference exactly on all but a small fraction.
(2) Index work, exact: what the fused kernel selects is bit for bit the operator's
selection on those scores (CPU oracle of the operator; slot for slot when there is no
second stage)."""

import pytest
import torch

from approx_topk import topk
from approx_topk.attention import score_topk, scores
from oracle import cpu_oracle as oracle
from tests.helper_funcs import assert_valid_selection


def test_score_topk_checks_come_before_any_native_call():
    q = torch.randn(2, 128).bfloat16()
    keys = torch.randn(2, 64, 128).bfloat16()
    with pytest.raises(ValueError):
        score_topk(q, keys, 4, k_mult=0)
    with pytest.raises(RuntimeError, match="float16 or both bfloat16"):
        score_topk(q.float(), keys.float(), 4)
    with pytest.raises(ValueError, match="keys must be"):
        score_topk(q, keys[:, :, :64], 4)
    with pytest.raises(NotImplementedError):
        score_topk(q[:, :32], keys[:, :, :32], 4)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        score_topk(q, keys, 4)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        scores(q, keys)


def test_oracle_reference_scores():
    g = torch.Generator().manual_seed(0)
    q = torch.randn(3, 64, generator=g).bfloat16()
    keys = torch.randn(3, 50, 64, generator=g).bfloat16()
    s = oracle.scores(q, keys, 0.125)
    assert s.dtype == torch.bfloat16 and s.shape == (3, 50)
    ref = ((keys.double() @ q.double().unsqueeze(-1)).squeeze(-1).float() * 0.125).bfloat16()
    assert torch.equal(s.view(torch.int16), ref.view(torch.int16))
    # a case small enough to follow by hand: exact products, no rounding anywhere
    q = torch.tensor([[1.0, 2.0] + [0.0] * 62]).half()
    keys = torch.zeros(1, 3, 64).half()
    keys[0, 0, 0], keys[0, 1, 1], keys[0, 2, :2] = 4.0, 3.0, torch.tensor([1.0, 1.0]).half()
    assert oracle.scores(q, keys, 0.5).tolist() == [[2.0, 3.0, 1.5]]


CASES = [
    # dtype, rows, n, d, k, j, k_mult
    (torch.bfloat16, 6, 4096, 128, 256, 4, 2), (torch.bfloat16, 3, 4096 + 77, 128, 64, 2, 1),
    (torch.float16, 5, 8192, 64, 128, 1, 4), (torch.float16, 2, 1000, 128, 21, 3, 1),      # 7 buckets: an odd count
    (torch.bfloat16, 2, 65 * 600 + 5, 64, 1200, 2, 1), (torch.float16, 1, 300 * 70, 128, 35, 1, 2),
]


def _ulp(x: torch.Tensor, dtype) -> torch.Tensor:
    """One unit in the last place of the 16-bit type at the magnitude of x (float tensor)."""
    mant = 7 if dtype == torch.bfloat16 else 10
    exp = torch.floor(torch.log2(x.abs().clamp_min(2.0 ** -14)))
    return torch.exp2(exp - mant)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,rows,n,d,k,j,k_mult", CASES)
def test_score_topk_selects_exactly_what_the_operator_selects_on_its_scores(dtype, rows, n, d, k, j, k_mult):
    g = torch.Generator(device="cuda").manual_seed(rows * n + d)
    q = torch.randn(rows, d, device="cuda", generator=g).to(dtype)
    keys = torch.randn(rows, n, d, device="cuda", generator=g).to(dtype)
    scale = d ** -0.5
    s = scores(q, keys, scale)
    # (1) float work, tolerance: one unit in the last place of the 16-bit score
    # (plus the float32 accumulation error, which is relative to the sum of the products'
    # magnitudes, not to a result that cancellation made small)
    ref = oracle.scores(q, keys, scale).float()
    diff = (s.float().cpu() - ref).abs()
    spread = ((q.float().abs().unsqueeze(1) @ keys.float().abs().transpose(-1, -2)).squeeze(1) * scale).cpu()
    tol = _ulp(ref, dtype) + spread * 2.0 ** -22
    assert bool((diff <= tol).all()), float((diff / tol).max())
    assert float((diff > 0).float().mean()) < 0.02
    # (2) index work, exact: the fused kernel against the operator's oracle on those scores
    v, i = score_topk(q, keys, k, j=j, k_mult=k_mult, scale=scale)
    ov, oi = oracle.topk(s.cpu(), k, j=j, k_mult=k_mult)
    assert_valid_selection(s, v, i, ov)
    if k_mult == 1:
        assert torch.equal(v.cpu().view(torch.int16), ov.view(torch.int16)) and torch.equal(i.cpu(), oi)
    # and against the operator itself run on those scores on the device
    tv, ti = topk(s, k, -1, j=j, k_mult=k_mult)
    assert_valid_selection(s, tv, ti, v)
    if k_mult == 1:
        zero = v == 0                         # a score of -0.0 comes back as +0.0 from the fused kernel
        assert torch.equal(torch.where(zero, torch.zeros_like(v), v).view(torch.int16),
                           torch.where(zero, torch.zeros_like(tv), tv).view(torch.int16)) and torch.equal(i, ti)


@pytest.mark.gpu
def test_score_topk_leading_dimensions_and_default_scale():
    g = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn(2, 3, 128, device="cuda", generator=g).bfloat16()
    keys = torch.randn(2, 3, 2048, 128, device="cuda", generator=g).bfloat16()
    v, i = score_topk(q, keys, 64, j=2)
    assert v.shape == (2, 3, 64) and i.shape == (2, 3, 64) and i.dtype == torch.int64
    s = scores(q, keys)
    assert s.shape == (2, 3, 2048) and s.dtype == torch.bfloat16
    ov, oi = oracle.topk(s.reshape(6, 2048).cpu(), 64, j=2)
    assert torch.equal(v.reshape(6, 64).cpu().view(torch.int16), ov.view(torch.int16))
    assert torch.equal(i.reshape(6, 64).cpu(), oi)
    # against a torch matrix product: one unit in the last place
    unfused = ((q.float().unsqueeze(-2) @ keys.float().transpose(-1, -2)).squeeze(-2) * 128 ** -0.5)
    assert bool(((s.float() - unfused).abs() <= _ulp(unfused, torch.bfloat16)).all())
