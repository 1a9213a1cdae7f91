"""Opt-in narrow output formats (int32 positions, packed 8-byte records): the same
selection as the default int64 path, pair for pair and in the same order."""

import pytest
import torch

from approx_topk import _native, topk
from approx_topk.formats import topk_narrow


def _bits32(v: torch.Tensor) -> torch.Tensor:
    """The element's bits zero-extended to 32 bits, as int32 (what a record holds)."""
    if v.element_size() == 4:
        return v.view(torch.int32)
    if v.element_size() == 2:
        return v.view(torch.int16).to(torch.int32) & 0xFFFF
    return v.view(torch.uint8).to(torch.int32)


# (dtype, rows, n, k, j, k_mult): one-stage write-outs of every vector width, the stripe split
# over blocks (plane merge writes the final pairs), the one-block select, its packed hand-off
# and the multi-block select.
CASES = [
    (torch.float32, 8, 1 << 16, 1 << 12, 2, 1), (torch.float32, 3, 10007, 33, 3, 1), (torch.float32, 5, 4096, 64, 1, 1),
    (torch.bfloat16, 8, 1 << 16, 1 << 12, 4, 1), (torch.float16, 4, 1 << 14, 512, 2, 1), (torch.float16, 3, 4099, 7, 1, 1),
    (torch.int16, 4, 1 << 14, 256, 2, 1), (torch.int8, 4, 1 << 14, 256, 1, 1), (torch.int32, 4, 1 << 14, 256, 4, 1),
    (torch.float32, 1, 1 << 20, 64, 2, 1), (torch.float16, 1, 1 << 20, 32, 4, 1),
    (torch.float32, 16, 1 << 14, 128, 2, 2), (torch.bfloat16, 64, 1 << 16, 2048, 4, 2), (torch.float16, 32, 128256, 64, 1, 4),
    (torch.float32, 2, 1 << 20, 1 << 14, 4, 2), (torch.bfloat16, 2, 1 << 20, 1 << 14, 2, 2),
]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,rows,n,k,j,k_mult", CASES, ids=[f"{c[0]}-{c[1]}x{c[2]}-k{c[3]}-j{c[4]}-m{c[5]}".replace("torch.", "") for c in CASES])
def test_narrow_formats_equal_the_int64_path(dtype, rows, n, k, j, k_mult):
    g = torch.Generator(device="cuda").manual_seed(rows + n + k)
    if dtype.is_floating_point:
        x = torch.randn(rows, n, device="cuda", generator=g).to(dtype)
    else:
        info = torch.iinfo(dtype)
        x = torch.randint(info.min, info.max, (rows, n), device="cuda", generator=g, dtype=torch.int64).to(dtype)
    v, i = topk(x, k, -1, j=j, k_mult=k_mult)
    nv, ni = topk_narrow(x, k, -1, j=j, k_mult=k_mult)
    assert ni.dtype == torch.int32 and nv.dtype == dtype
    assert torch.equal(_bits32(nv), _bits32(v)) and torch.equal(ni.to(torch.int64), i)
    rec = topk_narrow(x, k, -1, j=j, k_mult=k_mult, records=True)
    assert rec.shape == (rows, k, 2) and rec.dtype == torch.int32
    assert torch.equal(rec[..., 0], _bits32(v)) and torch.equal(rec[..., 1].to(torch.int64), i)
    # a strided input view and a 1-D row
    if rows > 1:
        xv = x[::2]
        sv, si = topk_narrow(xv, k, -1, j=j, k_mult=k_mult)
        assert torch.equal(_bits32(sv), _bits32(v[::2])) and torch.equal(si.to(torch.int64), i[::2])
    rv, ri = topk_narrow(x[0], k, -1, j=j, k_mult=k_mult)
    assert torch.equal(_bits32(rv), _bits32(v[0])) and torch.equal(ri.to(torch.int64), i[0])


@pytest.mark.gpu
def test_narrow_format_argument_checks():
    lib = _native.lib()
    x = torch.randn(2, 256, device="cuda")
    out = torch.empty(2, 16, 2, device="cuda", dtype=torch.int32)
    stream = torch.cuda.current_stream().cuda_stream

    def call(code, fmt, interleaved=1, n=256):
        return lib.atk_topk_ex(x.data_ptr(), code, 2, n, n, 16, 1, 1, interleaved, -1, fmt, out.data_ptr(),
                               out.data_ptr(), 16, None, 0, stream)

    assert call(0, 7) == _native.ATK_ERR_BAD_ARG                      # unknown format
    assert call(0, _native.ATK_OUT_I32, interleaved=0) == _native.ATK_ERR_BAD_ARG   # contiguous buckets
    assert call(3, _native.ATK_OUT_REC32) == _native.ATK_ERR_BAD_DTYPE              # float64 has no 32-bit record
    assert call(0, _native.ATK_OUT_I32, n=1 << 31) == _native.ATK_ERR_TOO_LARGE     # positions would not fit
    with pytest.raises(NotImplementedError):
        topk_narrow(x, 16, dim=0)
    with pytest.raises(ValueError):
        topk_narrow(x, 16, k_mult=0)


def test_narrow_format_checks_come_before_any_native_call():
    x = torch.randn(2, 64)
    with pytest.raises(NotImplementedError):
        topk_narrow(x, 4, dim=0)
    with pytest.raises(ValueError):
        topk_narrow(x, 4, k_mult=0)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        topk_narrow(x, 4)
