"""Bucketed approximate top-k for NVIDIA B200 (sm_100a).

Drop-in for the operator API of graphcore-research/pytorch-approx-topk:
``approx_topk.topk``, ``approx_topk.priority_queue.topk`` (the
``approx_topk::topk`` custom op) and ``approx_topk.experimental.*``.
"""

from typing import Protocol

from torch import Tensor

from .priority_queue import topk as topk


class Topk(Protocol):
    """Anything callable like ``torch.topk(xs, k, dim) -> (values, indices)``."""

    @staticmethod
    def __call__(xs: Tensor, k: int, dim: int) -> tuple[Tensor, Tensor]: ...
