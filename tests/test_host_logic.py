"""CPU-only checks: the C-ABI library loads and exports every symbol the header
declares, status texts, the Python operator's argument handling and meta
implementation, and the torch-composition helpers of approx_topk.experimental."""

import ctypes
import re
from pathlib import Path

import pytest
import torch

from approx_topk import Topk, _native, topk
from approx_topk.cuda_extensions import load_cuda_extension
from approx_topk.experimental.autobucket import bucket, bucketed_torch_topk
from approx_topk.experimental.bucketed_argmax import _batch_contiguous, _min_value, topk_torch, topk_triton
from tests.helper_funcs import assert_close_up_to_permutation

ROOT = Path(__file__).resolve().parents[1]


def declared_functions() -> list[str]:
    text = (ROOT / "include" / "atk.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"\b(atk_[a-z0-9_]+)\s*\(", text)


def test_library_exports_every_declared_symbol():
    names = declared_functions()
    assert len(names) >= 12
    handle = ctypes.CDLL(str(_native.library_path()))
    for name in names:
        assert hasattr(handle, name), f"libatk.so lacks {name}"
    assert set(names) == set(_native.SIGNATURES), "python prototypes and header differ"


def test_version_and_status_texts():
    lib = load_cuda_extension("priority_queue_approx_topk.cu", compile_mode="optimize")
    assert lib is _native.lib()
    assert lib.atk_version() >= 10000
    assert _native.strerror(0) == "ok"
    assert "j must divide k" in _native.strerror(_native.ATK_ERR_J_DIVIDES_K)
    assert "0 < j < 5" in _native.strerror(_native.ATK_ERR_BAD_J)
    assert "must not be larger" in _native.strerror(_native.ATK_ERR_K_TOO_LARGE)
    assert lib.atk_topk_workspace_bytes(0, 8, 4096, 64, 2, 1) == 0
    need = lib.atk_topk_workspace_bytes(0, 8, 4096, 64, 2, 4)
    assert need >= 8 * 256 * (4 + 8)
    assert lib.atk_select_workspace_bytes(0, 1, 1 << 21, 1 << 20) > 0
    assert lib.atk_select_workspace_bytes(2, 1024, 4096, 2048) == 0


def test_python_checks_come_before_any_native_call():
    xs = torch.randn(8, 64)
    with pytest.raises(NotImplementedError):
        topk(xs, 4, dim=0, j=2)
    with pytest.raises(ValueError):
        topk(xs, 4, dim=-1, k_mult=0)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        topk(xs, 4, dim=-1)          # no CPU path, and it says so
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        topk_torch(xs, 4, dim=-1, interleaved=True)
    with pytest.raises(ValueError):
        topk_triton(xs, 4, dim=-1, interleaved=True, block_size=8, kernel="nope")


def test_meta_implementation_shapes():
    xs = torch.empty(5, 7, 64, device="meta", dtype=torch.bfloat16)
    v, i = topk(xs, 8, -1, 2, 2)
    assert v.shape == (5, 7, 8) and v.dtype == torch.bfloat16 and v.device.type == "meta"
    assert i.shape == (5, 7, 8) and i.dtype == torch.int64
    v, i = topk(torch.empty(6, 4, device="meta"), 4, 0, 4)
    assert v.shape == (4, 4)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("ATK_LIBRARY", str(tmp_path / "nope.so"))
    _native.lib.cache_clear()
    try:
        with pytest.raises(RuntimeError, match="not found"):
            _native.lib()
    finally:
        monkeypatch.delenv("ATK_LIBRARY")
        _native.lib.cache_clear()
        _native.lib()


def test_as_rows_layouts():
    x = torch.arange(6 * 10.0).reshape(6, 10)
    t, rows, n, stride = _native.as_rows(x)
    assert t is x and (rows, n, stride) == (6, 10, 10)
    t, rows, n, stride = _native.as_rows(x[:, :8])
    assert t.data_ptr() == x.data_ptr() and (rows, n, stride) == (6, 8, 10)
    t, rows, n, stride = _native.as_rows(x[:, ::2])
    assert t.is_contiguous() and (rows, n, stride) == (6, 5, 5)
    y = torch.arange(2 * 3 * 4.0).reshape(2, 3, 4)
    t, rows, n, stride = _native.as_rows(y.movedim(0, -1))
    assert t.is_contiguous() and (rows, n, stride) == (12, 2, 2)


def test_min_value():
    assert _min_value(torch.float16) == -65504.0
    assert _min_value(torch.int16) == -32768


def test_batch_contiguous():
    x = torch.arange(3 * 4 * 5).view(3, 4, 5)
    for t, same in [(x, True), (x[:, :, :-1], True), (x[:, :, ::2], False), (x[:, :-1, :], False),
                    (x.swapdims(0, 1), False)]:
        t2 = _batch_contiguous(t)
        if same:
            assert t2 is t
        else:
            assert torch.equal(t, t2) and t2.is_contiguous()
        assert t2.stride(-1) == 1


# --- the generic bucketed construction (runs on CPU tensors) ----------------

def exact(xs, k, dim):
    return torch.topk(xs, k, dim, sorted=False)


def test_bucket_rejects_indivisible_k():
    with pytest.raises(NotImplementedError):
        bucket(exact, k_mult=1, k_per_bucket=12, interleaved=True)(torch.randn(1024), 13, dim=0)


@pytest.mark.parametrize("interleaved", [True, False])
def test_bucket_single_bucket_is_exact(interleaved):
    xs = torch.randn(1024)
    v, i = bucket(exact, k_mult=1, k_per_bucket=128, interleaved=interleaved)(xs, 128, dim=0)
    ev, ei = exact(xs, 128, 0)
    assert_close_up_to_permutation(v, ev)
    assert_close_up_to_permutation(i, ei)


@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("k_mult", [1, 2, 4])
@pytest.mark.parametrize("k_per_bucket", [1, 2, 4])
def test_bucket_shapes(interleaved, k_mult, k_per_bucket):
    v, i = bucketed_torch_topk(torch.randn(5, 32, 1000), 16, -1, k_mult, k_per_bucket, interleaved)
    assert v.shape == (5, 32, 16) and i.shape == (5, 32, 16)


@pytest.mark.parametrize("interleaved,k_mult,k,n,expected", [
    (False, 1, 3, 10, [3, 6, 9]), (True, 1, 3, 10, [9, 7, 8]),
    (False, 2, 4, 16, [15, 13, 11, 9]), (True, 2, 4, 16, [15, 14, 13, 12]),
])
def test_bucket_arange_cases(interleaved, k_mult, k, n, expected):
    v, i = bucket(torch.topk, k_mult=k_mult, k_per_bucket=1, interleaved=interleaved)(torch.arange(n), k=k, dim=-1)
    assert_close_up_to_permutation(v, torch.tensor(expected))
    assert_close_up_to_permutation(i, torch.tensor(expected))


def test_bucket_matches_reference_fixtures(golden):
    data, meta = golden
    for idx, m in enumerate(meta):
        if m["kind"] != "bucketed_torch_topk" or m["dtype"] != "float32":
            continue
        x = torch.from_numpy(data[f"c{idx}_x"])
        v, i = bucketed_torch_topk(x, m["k"], -1, m["k_mult"], m["j"], m["interleaved"])
        assert torch.equal(v.sort(dim=-1).values, torch.from_numpy(data[f"c{idx}_values"])), m
        assert torch.equal(i.sort(dim=-1).values, torch.from_numpy(data[f"c{idx}_indices"])), m


def test_topk_protocol_is_exported():
    assert hasattr(Topk, "__call__")


def test_bench_clock_sampler_degrades_without_a_gpu():
    # no driver here: neither NVML nor nvidia-smi answers, the summary says so instead of failing
    import importlib.util
    from pathlib import Path

    spec = importlib.util.spec_from_file_location("atk_bench_main", Path(__file__).resolve().parents[1] / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    with bench.ClockSampler(0) as sampler:
        pass
    summary = sampler.summary()
    assert summary["samples"] == 0 and summary["reasons"] == [] and summary["sm_mhz"] is None


def test_every_element_type_of_the_reference_dispatch_has_a_code():
    from approx_topk import _native

    want = {torch.float32, torch.float16, torch.bfloat16, torch.float64,
            torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8}
    assert set(_native.DTYPE_CODES) == want
    assert sorted(_native.DTYPE_CODES.values()) == list(range(9))
    with pytest.raises(RuntimeError, match="not supported"):
        _native.dtype_code(torch.bool)


def test_gather_checks_come_before_any_native_call():
    from approx_topk.gather import gather_records

    src = torch.ones(2, 10, 4)
    idx = torch.zeros(2, 3, dtype=torch.int64)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        gather_records(src, idx)            # no CPU path, and it says so


def test_reference_cpu_tests_pass_unmodified_against_this_package():
    # Where the reference checkout is present, its own CPU-runnable test files are
    # collected as they are and run against THIS package (the module paths are the
    # same).  The reference's GPU tests need both a GPU and the checkout, which are
    # never on one machine here; tests/test_priority_queue.py restates them.
    import os
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    ref = Path(os.environ.get("ATK_REFERENCE_ROOT", root.parent / "reference"))
    files = [ref / "tests" / "test_autobucket.py", ref / "tests" / "test_bucket_argmax.py"]
    if not all(f.exists() for f in files):
        pytest.skip("reference checkout not present on this machine")
    code = (
        "import sys, pytest, approx_topk\n"
        "assert 'pytorch-approx-topk_b200' in approx_topk.__file__, approx_topk.__file__\n"
        f"sys.exit(pytest.main(['-q', '-p', 'no:cacheprovider', '--rootdir', {str(root)!r}, "
        f"{str(files[0])!r}, {str(files[1]) + '::test_batch_contiguous'!r}]))\n"
    )
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([str(root), str(root / "pytorch-approx-topk_b200")]))
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=str(root), env=env,
                         timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert " passed" in res.stdout and "failed" not in res.stdout


def test_bench_reference_arm_prints_the_contract_line_with_the_gpu_arms_config():
    # the reference arm (CPU path on the host cores) must describe the same configuration as
    # the GPU arm does -- the two lines are compared key for key -- and carry the contract's keys
    import importlib.util
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    res = subprocess.run([sys.executable, str(root / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                          "--workload", "c4j1"], capture_output=True, text=True, timeout=900, cwd=str(root))
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    spec = importlib.util.spec_from_file_location("atk_bench_cfg", root / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert line["config"] == bench.config_of(bench.WORKLOADS["c4j1"], "c4j1")
    assert line["impl"] == "reference" and line["metric"] == bench.METRIC and line["unit"] == "rows/s"
    assert line["higher_is_better"] is True and line["gpu_launches"] == 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["value"] > 0 and abs(line["ms_per_step"] * line["value"] / 1e3 / 4096 - 1.0) < 1e-6


def test_bench_host_samples_follow_the_workloads_distribution():
    import importlib.util
    from pathlib import Path

    spec = importlib.util.spec_from_file_location("atk_bench_data", Path(__file__).resolve().parents[1] / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    # attention scores on the host: N(0, |q|^2 / 128) per row, in bf16
    x, k, scale = bench.cpu_sample(dict(bench.WORKLOADS["c3"], n=4096), 8)
    assert x.shape == (8, 4096) and x.dtype == torch.bfloat16 and k == 2048 and scale == 1
    assert 0.5 < float(x.float().std()) < 1.5
    # spikes: 16 positions per row stand 8 above the N(0, 2) body
    x, _, _ = bench.cpu_sample(dict(bench.WORKLOADS["c4j1"], n=8192), 4)
    assert x.dtype == torch.float16 and int((x.float() > 7.5).sum()) >= 4 * 8
    # the long row is sampled by a slice with the same bucket length
    w = bench.WORKLOADS["c5b"]
    n = 1 << 26
    assert w["n"] // n == 64 and max(w["k"] // 64, w["j"]) * w["k_mult"] // w["j"] * (w["n"] // (w["k"] * w["k_mult"] // w["j"])) == n


def test_push_exchange_argument_checks_need_no_gpu():
    """atk_push_blocks validates counts, null pointers and alignment before it touches CUDA;
    LongRowTopK rejects an unknown exchange before it touches the process group."""
    import ctypes

    from approx_topk import _native
    from approx_topk.distributed import LongRowTopK

    lib = _native.lib()
    src = (ctypes.c_void_p * 1)(256)
    nbytes = (ctypes.c_size_t * 1)(64)
    dst = (ctypes.c_void_p * 1)(512)
    assert lib.atk_push_blocks(0, src, nbytes, 1, dst, None) == _native.ATK_OK            # nothing to do
    assert lib.atk_push_blocks(1, src, nbytes, 0, dst, None) == _native.ATK_OK
    assert lib.atk_push_blocks(5, src, nbytes, 1, dst, None) == _native.ATK_ERR_BAD_ARG   # too many segments
    assert lib.atk_push_blocks(1, src, nbytes, 17, dst, None) == _native.ATK_ERR_BAD_ARG  # too many destinations
    assert lib.atk_push_blocks(1, None, nbytes, 1, dst, None) == _native.ATK_ERR_BAD_ARG
    odd = (ctypes.c_size_t * 1)(6)
    assert lib.atk_push_blocks(1, src, odd, 1, dst, None) == _native.ATK_ERR_BAD_ARG      # not a multiple of 4 bytes
    unaligned = (ctypes.c_void_p * 1)(514)
    assert lib.atk_push_blocks(1, src, nbytes, 1, unaligned, None) == _native.ATK_ERR_BAD_ARG
    null_dst = (ctypes.c_void_p * 1)(None)
    assert lib.atk_push_blocks(1, src, nbytes, 1, null_dst, None) == _native.ATK_ERR_BAD_ARG
    assert lib.atk_peer_alloc(0, None, None) == _native.ATK_ERR_BAD_ARG
    assert lib.atk_peer_open(None, None) == _native.ATK_ERR_BAD_ARG
    assert lib.atk_peer_close(None) == _native.ATK_OK and lib.atk_peer_free(None) == _native.ATK_OK
    with pytest.raises(ValueError, match="exchange"):
        LongRowTopK(16, 8, 1, 1, torch.float32, torch.device("cpu"), exchange="carrier pigeon")


def test_peer_buffer_failures_are_raised_on_every_rank_alike():
    """PeerBuffers gathers every rank's outcome before it goes on: whichever rank failed, all
    ranks release what they hold (the release holds a barrier, so all must enter it) and raise
    the same error."""
    from approx_topk.distributed import PeerBuffers

    released = []
    pb = object.__new__(PeerBuffers)
    pb._release = lambda: released.append(True)
    pb._raise_together([None, None, None])              # nobody failed: nothing happens
    assert released == []
    with pytest.raises(RuntimeError, match=r"rank 1: no peer access.*rank 2: cannot map"):
        pb._raise_together([None, "no peer access", "cannot map"])
    assert released == [True]
