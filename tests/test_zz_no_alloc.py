"""GPU test of ``atk_select_static`` — the exact select for callers that cannot
allocate device memory.

Some users of the library cannot create the workspace that ``atk_select``
wants: a plugin inside a server that owns the whole GPU memory budget, a loop
that must not risk a device-wide stall from ``cudaMalloc``, or code that only
has raw pointers and a stream from another runtime.  For them the library
carries 1 MiB of scratch inside its own image and ``atk_select_static`` uses
that instead of a workspace argument.

The test calls the new entry point through the C ABI, twice in a row on
problems that really use the scratch (more than 16384 candidates per row) and
of different sizes, so the second call runs over whatever the first one left
in the shared array, and requires bit-identical results to ``atk_select``.
It also checks that a problem beyond the 1 MiB limit is refused with a clear
error and launches nothing.  The file sorts last so that a run that stops at
the first failure has already run every other test; it also passes on its own
in a fresh process (the first call does the per-device set-up itself).
"""

import pytest
import torch

from approx_topk import _native

pytestmark = pytest.mark.gpu


def _select(entry: str, cand_vals: torch.Tensor, cand_idx: torch.Tensor, k: int):
    rows, k0 = cand_vals.shape
    code = _native.dtype_code(cand_vals.dtype)
    lib = _native.lib()
    vals = torch.full((rows, k), float("nan"), device=cand_vals.device, dtype=cand_vals.dtype)
    idx = torch.full((rows, k), -7, device=cand_vals.device, dtype=torch.int64)
    stream = torch.cuda.current_stream(cand_vals.device).cuda_stream
    if entry == "static":
        rc = lib.atk_select_static(cand_vals.data_ptr(), cand_idx.data_ptr(), code, rows, k0, k0, k,
                                   vals.data_ptr(), idx.data_ptr(), k, stream)
    else:
        nbytes = lib.atk_select_workspace_bytes(code, rows, k0, k)
        ws = torch.empty(max(nbytes, 1), device=cand_vals.device, dtype=torch.uint8)
        rc = lib.atk_select(cand_vals.data_ptr(), cand_idx.data_ptr(), code, rows, k0, k0, k,
                            vals.data_ptr(), idx.data_ptr(), k, ws.data_ptr() if nbytes else None, nbytes, stream)
    return rc, vals, idx


def _candidates(rows, k0, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    vals = torch.randn(rows, k0, device="cuda", generator=g).to(dtype)
    idx = torch.randperm(rows * k0, device="cuda", generator=g).reshape(rows, k0)
    return vals, idx


def test_static_scratch_select_matches_workspace_select_on_two_calls_in_a_row():
    lib = _native.lib()
    # both problems take the multi-block path, i.e. they use the scratch
    problems = [(3, 100_000, 40_000, torch.float32, 1), (1, 1 << 21, 1 << 20, torch.float32, 2),
                (2, 70_001, 123, torch.bfloat16, 3)]
    for rows, k0, k, dtype, seed in problems:
        assert 0 < lib.atk_select_workspace_bytes(_native.dtype_code(dtype), rows, k0, k) <= (1 << 20)
    inputs = [_candidates(rows, k0, dtype, seed) for rows, k0, k, dtype, seed in problems]
    # two (here three) calls back to back on one stream, no synchronisation between them
    got = [_select("static", cv, ci, p[2]) for (cv, ci), p in zip(inputs, problems)]
    want = [_select("workspace", cv, ci, p[2]) for (cv, ci), p in zip(inputs, problems)]
    torch.cuda.synchronize()
    for (rc_s, v_s, i_s), (rc_w, v_w, i_w) in zip(got, want):
        assert rc_s == 0 and rc_w == 0
        # integer / bit-exact work: no tolerance
        assert torch.equal(v_s.view(torch.int16 if v_s.element_size() == 2 else torch.int32),
                           v_w.view(torch.int16 if v_w.element_size() == 2 else torch.int32))
        assert torch.equal(i_s, i_w)
    # and once more over the state the previous calls left behind
    rc, v, i = _select("static", *inputs[0], problems[0][2])
    torch.cuda.synchronize()
    assert rc == 0 and torch.equal(v, want[0][1]) and torch.equal(i, want[0][2])


def test_static_scratch_select_small_rows_need_no_scratch():
    cv, ci = _candidates(16, 4096, torch.float16, 9)
    rc_s, v_s, i_s = _select("static", cv, ci, 2048)
    rc_w, v_w, i_w = _select("workspace", cv, ci, 2048)
    torch.cuda.synchronize()
    assert rc_s == 0 and rc_w == 0
    assert torch.equal(v_s.view(torch.int16), v_w.view(torch.int16)) and torch.equal(i_s, i_w)


def test_static_scratch_select_refuses_what_does_not_fit():
    lib = _native.lib()
    rows, k0, k = 4096, 40_000, 10           # 4096 rows x (state + histograms + counts) > 1 MiB
    assert lib.atk_select_workspace_bytes(0, rows, k0, k) > (1 << 20)
    # nothing may be launched or written: the buffers are tiny sentinels
    cv = torch.zeros(1, device="cuda")
    ci = torch.zeros(1, device="cuda", dtype=torch.int64)
    out_v = torch.full((4,), 5.0, device="cuda")
    out_i = torch.full((4,), 5, device="cuda", dtype=torch.int64)
    rc = lib.atk_select_static(cv.data_ptr(), ci.data_ptr(), 0, rows, k0, k0, k, out_v.data_ptr(),
                               out_i.data_ptr(), k, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == _native.ATK_ERR_SCRATCH_LIMIT
    assert "atk_select_static" in _native.strerror(rc) and "1 MiB" in _native.strerror(rc)
    assert bool((out_v == 5.0).all()) and bool((out_i == 5).all())
