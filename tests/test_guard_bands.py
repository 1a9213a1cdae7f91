"""Out-of-bounds detection without a sanitizer: inputs sit between guard bands of
+inf (any read outside a row's extent would win the selection and show up as a
mismatch with the oracle) and outputs sit between guard bands of a sentinel
that must survive every call.  Exhaustive over small shapes, all legal
(k0, j) for each n, both bucket layouts, unaligned bases included."""

import pytest
import torch

from approx_topk import _native
from oracle import cpu_oracle as oracle

pytestmark = pytest.mark.gpu

GUARD = 64


def run_guarded(x_cpu: torch.Tensor, k: int, j: int, k_mult: int, interleaved: bool, shift: int):
    rows, n = x_cpu.shape
    dtype = x_cpu.dtype
    lib = _native.lib()
    code = _native.dtype_code(dtype)
    # input: [guard + shift | rows*n | guard], +inf outside the rows
    buf = torch.full((GUARD + shift + rows * n + GUARD,), float("inf"), device="cuda", dtype=dtype)
    x = buf[GUARD + shift:GUARD + shift + rows * n].view(rows, n)
    x.copy_(x_cpu)
    vbuf = torch.full((GUARD + rows * k + GUARD,), -12345.0, device="cuda", dtype=dtype)
    ibuf = torch.full((GUARD + rows * k + GUARD,), -777, device="cuda", dtype=torch.int64)
    v = vbuf[GUARD:GUARD + rows * k].view(rows, k)
    i = ibuf[GUARD:GUARD + rows * k].view(rows, k)
    ws_bytes = lib.atk_topk_workspace_bytes(code, rows, n, k, j, k_mult)
    ws = torch.empty(max(ws_bytes, 1), device="cuda", dtype=torch.uint8)
    rc = lib.atk_topk(x.data_ptr(), code, rows, n, n, k, j, k_mult, int(interleaved), -1, v.data_ptr(),
                      i.data_ptr(), k, ws.data_ptr() if ws_bytes else None, ws_bytes,
                      torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _native.strerror(rc)
    torch.cuda.synchronize()
    for band in (vbuf[:GUARD], vbuf[-GUARD:]):
        assert bool((band == -12345.0).all()), "value output written outside its extent"
    for band in (ibuf[:GUARD], ibuf[-GUARD:]):
        assert bool((band == -777).all()), "index output written outside its extent"
    return v.cpu(), i.cpu()


def check(x_cpu, k, j, k_mult, interleaved, shift):
    v, i = run_guarded(x_cpu, k, j, k_mult, interleaved, shift)
    ov, oi = oracle.topk(x_cpu, k, j=j, k_mult=k_mult, interleaved=interleaved)
    assert bool(torch.isfinite(v.float()).all()), "a guard element was selected (read outside the row)"
    assert bool(((i >= 0) & (i < x_cpu.shape[-1])).all())
    assert torch.equal(v.float().sort(-1).values, ov.float().sort(-1).values)
    assert torch.equal(x_cpu.gather(-1, i), v)
    if x_cpu.dtype == torch.float32:
        assert torch.equal(i.sort(-1).values, oi.sort(-1).values)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [True, False])
def test_exhaustive_small_shapes(dtype, interleaved):
    g = torch.Generator().manual_seed(5)
    cases = 0
    for n in list(range(1, 41)) + [63, 64, 65, 96, 127, 128, 129]:
        x = torch.randn(3, n, generator=g).to(dtype)
        for j in (1, 2, 3, 4):
            for b in range(1, n // j + 1):
                if n > 40 and b not in (1, 2, 3, 4, 7, 8, 16, n // j):
                    continue
                check(x, b * j, j, 1, interleaved, shift=(cases % 3))
                cases += 1
    assert cases > 500


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_two_stage_and_split_shapes_between_guards(dtype):
    g = torch.Generator().manual_seed(6)
    for rows, n, k, j, k_mult, shift in [(2, 1000, 16, 2, 4, 1), (1, 300001, 32, 4, 2, 3), (5, 4099, 64, 1, 2, 0),
                                         (1, 1 << 20, 16, 2, 1, 2), (3, 70000, 1000, 4, 2, 5), (1, 65537, 4, 4, 1, 7)]:
        x = torch.randn(rows, n, generator=g).to(dtype)
        check(x, k, j, k_mult, True, shift)
