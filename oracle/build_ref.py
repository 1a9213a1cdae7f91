"""Recipe that compiles the reference's CUDA operator into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  The product never imports anything from here.

The reference ships one CUDA translation unit
(``approx_topk/priority_queue_approx_topk.cu``, pybind entry point
``PriorityQueueTopK`` at lines 378-387 / 523-525) that it JIT-compiles on first
use (``approx_topk/cuda_extensions.py:12-27``).  This script compiles that file
*where it lies* in the read-only reference checkout with a single ``nvcc``
command (no copy of the source is made, the reference's own loader is not run)
and writes only the resulting extension module
``oracle/_ref/atk_reference_cuda.so``.  The module needs a GPU to execute, so it
is only ever called from ``-m gpu`` parity tests (which fail when the file is
absent) and from the "reference_cuda" baseline leg of ``bench.py`` (which
reports the absence instead of a time).

Usage:  python oracle/build_ref.py [--reference-root DIR] [--force]
The compile takes several minutes (hundreds of template instantiations).
"""

from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
MODULE_NAME = "atk_reference_cuda"
REL_SOURCE = Path("approx_topk") / "priority_queue_approx_topk.cu"


def output_path() -> Path:
    return OUT_DIR / f"{MODULE_NAME}.so"


def build(reference_root: Path, force: bool = False, verbose: bool = True) -> Path | None:
    """Compile the reference CUDA file; returns the .so path or None if the
    reference checkout is not present (e.g. on a machine that only received the
    prebuilt file)."""
    src = reference_root / REL_SOURCE
    out = output_path()
    if not src.exists():
        return out if out.exists() else None
    if out.exists() and not force and out.stat().st_mtime >= src.stat().st_mtime:
        return out

    from torch.utils import cpp_extension  # heavy import, keep local

    OUT_DIR.mkdir(parents=True, exist_ok=True)
    inc = cpp_extension.include_paths("cuda") + [sysconfig.get_paths()["include"]]
    lib = cpp_extension.library_paths("cuda")
    cmd = ["nvcc", "-shared", "-Xcompiler", "-fPIC", "-std=c++17", "-O3",
           "--generate-line-info", "--expt-relaxed-constexpr",
           # Same arch flags torch's JIT loader would pick for a B200 when the
           # reference is built by its own loader (generic sm_100 code).
           "-gencode", "arch=compute_100,code=sm_100",
           f"-DTORCH_EXTENSION_NAME={MODULE_NAME}",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1",
           "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
           "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__"]
    cmd += [f"-I{p}" for p in inc]
    cmd += [str(src), "-o", str(out)]
    cmd += [f"-L{p}" for p in lib]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python"]
    cmd += [f"-Xlinker=-rpath={p}" for p in lib]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-root", default=os.environ.get("ATK_REFERENCE_ROOT", str(HERE.parents[1] / "reference")))
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    out = build(Path(args.reference_root), force=args.force)
    print("reference CUDA module:", out)
    return 0 if out is not None else 1


if __name__ == "__main__":
    sys.exit(main())
