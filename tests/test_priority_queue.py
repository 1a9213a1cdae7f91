"""GPU acceptance tests of ``approx_topk.topk`` — the cases the reference's
tests/test_priority_queue.py covers (one bucket, bucket size one, ideally
distributed inputs, equality with the generic bucketed construction, opcheck,
torch.compile), written against this package."""

import pytest
import torch
from torch import Generator

from approx_topk import topk as topk_export
from approx_topk.experimental.autobucket import bucketed_torch_topk
from approx_topk.priority_queue import topk
from tests.helper_funcs import assert_close_up_to_permutation

pytestmark = pytest.mark.gpu

ALL_DTYPES = [torch.float32, torch.bfloat16, torch.float16]
MODES = [False, True]


def rng_kwargs(seed: int):
    return dict(generator=Generator(device="cuda").manual_seed(seed), device="cuda")


def assert_same_selection(values, indices, expected_values, expected_indices, dim=-1):
    assert torch.allclose(values.sort(dim).values, expected_values.sort(dim).values)
    assert torch.allclose(indices.sort(dim).values, expected_indices.sort(dim).values)


def test_export_is_the_custom_op():
    assert topk_export is topk
    assert topk._opoverload.name() == "approx_topk::topk"


@pytest.mark.parametrize("k", [0, 2, 4])
@pytest.mark.parametrize("dtype", ALL_DTYPES)
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("multithread_buckets", MODES)
def test_one_bucket_1d_equals_exact(k, dtype, interleaved, multithread_buckets):
    xs = torch.randn(1001, dtype=dtype, **rng_kwargs(234))
    values, indices = topk(xs, k, j=k, dim=0, interleaved=interleaved,
                           multithread_buckets=multithread_buckets)
    ev, ei = torch.topk(xs, k, dim=0)
    assert values.dtype == dtype and indices.dtype == torch.int64
    assert values.shape == (k,) and indices.shape == (k,)
    assert torch.allclose(values.sort().values, ev.sort().values)
    if dtype == torch.float32:
        assert torch.equal(indices.sort().values, ei.sort().values)
    else:  # 16-bit rows can tie at the boundary: indices must point at the values
        assert torch.equal(xs[indices], values)


@pytest.mark.parametrize("k", [0, 2, 4])
@pytest.mark.parametrize("dim", [0, 1, 2])
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("multithread_buckets", MODES)
def test_one_bucket_batched_any_dim_equals_exact(k, dim, interleaved, multithread_buckets):
    xs = torch.rand((30, 25, 16), **rng_kwargs(4242))
    values, indices = topk(xs, k, j=k, dim=dim, interleaved=interleaved,
                           multithread_buckets=multithread_buckets)
    ev, ei = torch.topk(xs, k, dim)
    assert values.shape == ev.shape and values.is_contiguous()
    assert_same_selection(values, indices, ev, ei, dim)


@pytest.mark.parametrize("dim", [-1, -2])
def test_negative_dim(dim):
    xs = torch.randn((128, 256), **rng_kwargs(99))
    values, indices = topk(xs, k=4, j=4, dim=dim)
    ev, ei = torch.topk(xs, 4, dim)
    assert_same_selection(values, indices, ev, ei, dim)


def test_call_twice_same_result():
    xs = torch.randn((128,), **rng_kwargs(56))
    a = topk(xs, k=4, dim=0)
    b = topk(xs, k=4, dim=0)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


@pytest.mark.parametrize("n", [10, 16])
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("multithread_buckets", MODES)
def test_bucket_size_one_1d_is_exact(n, interleaved, multithread_buckets):
    xs = torch.randn(n, **rng_kwargs(856))
    values, indices = topk(xs, n, 0, j=1, interleaved=interleaved, multithread_buckets=multithread_buckets)
    ev, ei = torch.topk(xs, n, dim=0)
    assert_same_selection(values, indices, ev, ei, 0)


@pytest.mark.parametrize("dtype", ALL_DTYPES)
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("multithread_buckets", MODES)
def test_bucket_size_one_batched_is_exact(dtype, interleaved, multithread_buckets):
    xs = torch.randn((16, 4, 12), dtype=dtype, **rng_kwargs(23))
    dim = 2
    k = xs.size(dim)
    values, indices = topk(xs, k, dim, j=1, interleaved=interleaved, multithread_buckets=multithread_buckets)
    ev, ei = torch.topk(xs, k, dim)
    assert_same_selection(values, indices, ev, ei, dim)


@pytest.mark.parametrize("dtype", ALL_DTYPES)
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("multithread_buckets", MODES)
def test_k_mult_gives_bucket_size_one_is_exact(dtype, interleaved, multithread_buckets):
    xs = torch.randn((32, 1024), dtype=dtype, **rng_kwargs(23))
    values, indices = topk(xs, 64, -1, k_mult=16, j=1, interleaved=interleaved,
                           multithread_buckets=multithread_buckets)
    ev, ei = torch.topk(xs, 64, -1)
    assert torch.allclose(values.sort(-1).values, ev.sort(-1).values)
    assert torch.equal(xs.gather(-1, indices), values)
    if dtype == torch.float32:
        assert torch.equal(indices.sort(-1).values, ei.sort(-1).values)


@pytest.mark.parametrize("multithread_buckets", MODES)
def test_contiguous_ideally_distributed_n17(multithread_buckets):
    # 4 buckets over 17 positions: [0..4] [5..8] [9..12] [13..16], two per bucket
    xs = torch.zeros((2, 17), device="cuda")
    xs[0, [0, 4, 5, 8, 9, 12, 13, 16]] = torch.arange(11.0, 19.0, device="cuda")
    xs[1, [2, 3, 6, 7, 10, 11, 14, 15]] = torch.arange(21.0, 29.0, device="cuda")
    values, indices = topk(xs, 8, dim=1, j=2, interleaved=False, multithread_buckets=multithread_buckets)
    ev, ei = torch.topk(xs, 8, dim=1)
    assert_same_selection(values, indices, ev, ei, 1)


@pytest.mark.parametrize("multithread_buckets", MODES)
def test_contiguous_ideally_distributed_long(multithread_buckets):
    n, stride = 10_000, 625
    xs = torch.zeros((2, n), device="cuda")
    for r, first in ((0, 0), (1, 50)):
        pos = torch.arange(first, n, stride, device="cuda")
        vals = torch.rand(len(pos), **rng_kwargs(1)) + 2.0
        vals[(torch.arange(len(pos), device="cuda") % 4) < 2] += 1.0
        xs[r, pos] = vals
    values, indices = topk(xs, 8, dim=1, j=2, interleaved=False, multithread_buckets=multithread_buckets)
    ev, ei = torch.topk(xs, 8, dim=1)
    assert_same_selection(values, indices, ev, ei, 1)


@pytest.mark.parametrize("multithread_buckets", MODES)
def test_interleaved_ideally_distributed_n17(multithread_buckets):
    # interleaved buckets [0 4 8 12 16] [1 5 9 13] [2 6 10 14] [3 7 11 15]
    xs = torch.zeros((2, 17), device="cuda")
    xs[0, [0, 16, 1, 13, 2, 14, 3, 15]] = torch.arange(11.0, 19.0, device="cuda")
    xs[1, [4, 8, 5, 9, 6, 10, 7, 11]] = torch.arange(21.0, 29.0, device="cuda")
    values, indices = topk(xs, 8, dim=1, j=2, interleaved=True, multithread_buckets=multithread_buckets)
    ev, ei = torch.topk(xs, 8, dim=1)
    assert_same_selection(values, indices, ev, ei, 1)


@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("k_per_bucket", [1, 2, 4])
@pytest.mark.parametrize("multithread_buckets", MODES)
def test_equals_generic_bucketed_construction(interleaved, k_per_bucket, multithread_buckets):
    torch.manual_seed(100)
    xs = torch.randn(5, 32, 512, device="cuda")
    values, indices = topk(xs, k=64, dim=-1, j=k_per_bucket, interleaved=interleaved,
                           multithread_buckets=multithread_buckets)
    ev, ei = bucketed_torch_topk(xs, k=64, dim=-1, k_mult=1, k_per_bucket=k_per_bucket,
                                 interleaved=interleaved)
    assert_close_up_to_permutation(values, ev)
    assert_close_up_to_permutation(indices, ei)


@pytest.mark.parametrize("dtype", ALL_DTYPES)
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("multithread_buckets", [None, False, True])
def test_opcheck(dtype, interleaved, multithread_buckets):
    xs = torch.randn(32, 128, dtype=dtype, **rng_kwargs(0))
    torch.library.opcheck(
        topk, args=(xs,),
        kwargs=dict(k=12, dim=-1, j=1, interleaved=interleaved, multithread_buckets=multithread_buckets),
    )


compiled_topk = torch.compile(topk, fullgraph=True)


@pytest.mark.parametrize("dtype", ALL_DTYPES)
@pytest.mark.parametrize("interleaved", [False, True])
def test_torch_compile_equals_eager(dtype, interleaved):
    xs = torch.randn(32, 128, dtype=dtype, **rng_kwargs(0))
    kwargs = dict(xs=xs, k=12, dim=-1, j=2, interleaved=interleaved, multithread_buckets=None)
    ev, ei = topk(**kwargs)
    cv, ci = compiled_topk(**kwargs)
    assert torch.equal(ev, cv) and torch.equal(ei, ci)


def test_cuda_graph_capture_replays():
    xs = torch.randn(64, 4096, **rng_kwargs(5))
    topk(xs, 64, -1, j=2, k_mult=2)  # warm-up outside capture
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        v, i = topk(xs, 64, -1, j=2, k_mult=2)
    xs.copy_(torch.randn(64, 4096, **rng_kwargs(6)))
    g.replay()
    torch.cuda.synchronize()
    ev, ei = topk(xs, 64, -1, j=2, k_mult=2)
    assert torch.equal(v, ev) and torch.equal(i, ei)


def test_error_behaviour():
    xs = torch.randn(8, 64, device="cuda")
    with pytest.raises(NotImplementedError):
        topk(xs, 4, dim=0, j=2)                       # several buckets off the last dim
    with pytest.raises(ValueError):
        topk(xs, 4, dim=-1, k_mult=0)
    with pytest.raises(RuntimeError, match="j must divide k"):
        topk(xs, 6, dim=-1, j=4)
    with pytest.raises(RuntimeError, match="0 < j < 5"):
        topk(xs, 10, dim=-1, j=5)
    with pytest.raises(RuntimeError, match="must not be larger"):
        topk(xs, 128, dim=-1, j=1)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        topk(xs.cpu(), 4, dim=-1)
    with pytest.raises(RuntimeError, match="not supported"):
        topk(xs > 0, 4, dim=-1)


def test_non_contiguous_inputs():
    base = torch.randn(16, 300, **rng_kwargs(3))
    view = base[:, :256]                    # row stride 300, length 256
    a = topk(view, 32, -1, j=2)
    b = topk(view.contiguous(), 32, -1, j=2)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    strided = base[:, ::2]                  # element stride 2: copied
    a = topk(strided, 30, -1, j=2)
    b = topk(strided.contiguous(), 30, -1, j=2)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_runs_on_the_current_side_stream():
    # the kernels must be queued on torch's current stream, not the default one
    xs = torch.randn(64, 1 << 16, **rng_kwargs(8))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        big = torch.randn(1 << 26, device="cuda")       # keeps the side stream busy first
        ys = xs * 2.0                                    # produced on the side stream
        v, i = topk(ys, 128, -1, j=2, k_mult=2)
    side.synchronize()
    ev, ei = topk(xs * 2.0, 128, -1, j=2, k_mult=2)
    assert torch.equal(v, ev) and torch.equal(i, ei)
    del big


def test_host_buffer_python_api():
    from approx_topk.host_buffers import topk_host

    x = torch.randn(19, 4096, **rng_kwargs(9)).bfloat16()
    v, i = topk(x, 64, -1, j=4, k_mult=2)
    hv, hi = topk_host(x.cpu().pin_memory(), 64, j=4, k_mult=2)
    assert not hv.is_cuda and hv.is_pinned()
    assert torch.equal(hv, v.cpu()) and torch.equal(hi, i.cpu())
    out = (torch.empty(19, 64, dtype=torch.bfloat16), torch.empty(19, 64, dtype=torch.int64))
    rv, ri = topk_host(x.cpu(), 64, j=4, k_mult=2, out=out, chunk_rows=4)
    assert rv is out[0] and torch.equal(rv, v.cpu()) and torch.equal(ri, i.cpu())
    with pytest.raises(RuntimeError, match="CPU tensor"):
        topk_host(x, 64)
    with pytest.raises(ValueError):
        topk_host(x.cpu(), 64, out=(torch.empty(3, 3), torch.empty(3, 3, dtype=torch.int64)))
