"""Bucketed approximate top-k for NVIDIA B200 (sm_100a).

Drop-in for the operator API of graphcore-research/pytorch-approx-topk:
``approx_topk.topk``, ``approx_topk.priority_queue.topk`` (the
``approx_topk::topk`` custom op) and ``approx_topk.experimental.*``; plus
``approx_topk.host_buffers`` and ``approx_topk.distributed``.
"""

from __future__ import annotations

import typing

import torch

from . import priority_queue

__all__ = ["topk", "Topk"]

#: The operator, ``topk(xs, k, dim, j=1, k_mult=1, interleaved=True, multithread_buckets=False)``.
topk = priority_queue.topk


class Topk(typing.Protocol):
    """Structural type of anything callable like ``torch.topk``:
    ``f(xs, k, dim) -> (values, indices)``."""

    def __call__(self, xs: torch.Tensor, k: int, dim: int) -> tuple[torch.Tensor, torch.Tensor]:
        raise NotImplementedError
