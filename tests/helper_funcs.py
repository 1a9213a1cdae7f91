"""Comparison helpers shared by the tests (test infrastructure)."""

from __future__ import annotations

import torch
from torch import Tensor


def assert_close_up_to_permutation(x: Tensor, y: Tensor, dim: int = -1) -> None:
    """Equal as multisets along `dim` (the operator's output order is unspecified)."""
    torch.testing.assert_close(x.sort(dim=dim).values, y.sort(dim=dim).values)


def widen(t: Tensor) -> Tensor:
    """CPU copy in a type that holds every value of `t` exactly: float32 for the
    float types of 32 bits or fewer, float64 for float64, int64 for integers."""
    if t.dtype == torch.float64:
        wide = torch.float64
    else:
        wide = torch.float32 if t.dtype.is_floating_point else torch.int64
    return t.detach().to("cpu").to(wide)


def _bits(t: Tensor) -> Tensor:
    """Integer view of a widened tensor, so that comparisons are bit-exact."""
    if t.dtype == torch.float32:
        return t.view(torch.int32)
    if t.dtype == torch.float64:
        return t.view(torch.int64)
    return t


def assert_pairs_identical(values: Tensor, indices: Tensor, ref_values: Tensor, ref_indices: Tensor) -> None:
    """Bit-exact agreement of the selected (value, index) pairs per row after the
    canonical sort (value descending, then index ascending)."""
    from oracle.cpu_oracle import canonical

    v, i = canonical(values, indices)
    rv, ri = canonical(ref_values, ref_indices)
    assert torch.equal(_bits(v), _bits(rv)), "selected values differ"
    assert torch.equal(i, ri), "selected indices differ"


def assert_valid_selection(x: Tensor, values: Tensor, indices: Tensor, ref_values: Tensor) -> None:
    """Tie-tolerant acceptance rule: the value multiset matches the reference's,
    every returned index points at its value, and indices are distinct per row."""
    x2 = widen(x).reshape(-1, x.shape[-1])
    v = widen(values).reshape(x2.shape[0], -1)
    i = indices.detach().to("cpu").reshape(x2.shape[0], -1)
    rv = widen(ref_values).reshape(x2.shape[0], -1)
    assert torch.equal(v.sort(dim=-1).values, rv.sort(dim=-1).values), "value multiset differs"
    assert torch.equal(x2.gather(-1, i), v), "an index does not point at its value"
    si = i.sort(dim=-1).values
    assert bool((si[:, 1:] != si[:, :-1]).all()), "duplicate indices in a row"
