"""Builds libatk.so (the C-ABI library of the approximate top-k kernels) for sm_100a.

Plain nvcc, no JIT and no torch involvement: every translation unit under
``csrc/`` is compiled in parallel and linked into
``approx_topk/lib/libatk.so`` next to the Python host package.

Usage:  python build.py [--force] [--verbose] [-D NAME[=VALUE] ...]
"""

from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
INCLUDE = HERE.parent / "include"
OBJ_DIR = HERE / "build"
LIB_DIR = HERE / "approx_topk" / "lib"
LIB_PATH = LIB_DIR / "libatk.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    f"-I{INCLUDE}", f"-I{CSRC}",
]


def _newest_header_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in hdrs)


def _compile(src: Path, obj: Path, extra: list[str], verbose: bool) -> str:
    cmd = ["nvcc", *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    return res.stderr


def build(force: bool = False, verbose: bool = False, defines: list[str] | None = None) -> Path:
    extra = [f"-D{d}" for d in (defines or [])]
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    hdr_time = _newest_header_mtime()
    stamp = OBJ_DIR / "flags.txt"
    flags_text = " ".join(NVCC_FLAGS + extra)
    if not stamp.exists() or stamp.read_text() != flags_text:
        force = True
    jobs = []
    for src in sources:
        obj = OBJ_DIR / (src.stem + ".o")
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time)
        if stale:
            jobs.append((src, obj))
    logs = []
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            futs = [pool.submit(_compile, s, o, extra, verbose) for s, o in jobs]
            for f in futs:
                logs.append(f.result())
    objs = [OBJ_DIR / (s.stem + ".o") for s in sources]
    if jobs or not LIB_PATH.exists():
        cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", str(LIB_PATH), *map(str, objs)]
        subprocess.run(cmd, check=True)
    stamp.write_text(flags_text)
    if verbose:
        print("\n".join(logs))
    return LIB_PATH


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register / spill report")
    ap.add_argument("-D", dest="defines", action="append", default=[])
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.defines))
    return 0


if __name__ == "__main__":
    sys.exit(main())
