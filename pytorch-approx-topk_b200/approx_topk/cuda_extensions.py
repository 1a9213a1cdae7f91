"""Loader of the native kernels.

The reference JIT-compiles its CUDA file on first use through
``torch.utils.cpp_extension.load`` (reference approx_topk/cuda_extensions.py:12-27),
which costs minutes of nvcc time.  Here the kernels are prebuilt into
``lib/libatk.so`` by ``build.py`` and this function only opens that library, so
the name and signature are kept for callers that import it.
"""

from __future__ import annotations

import ctypes
from typing import Literal

from . import _native

CompileMode = Literal["default", "optimize", "debug"]


def load_cuda_extension(file_name: str = "priority_queue_approx_topk.cu",
                        compile_mode: CompileMode = "optimize") -> ctypes.CDLL:
    """Return the handle of the prebuilt C-ABI library (cached).

    ``file_name`` and ``compile_mode`` are accepted for signature compatibility;
    there is a single optimised build with line info.
    """
    if compile_mode not in ("default", "optimize", "debug"):
        raise ValueError(f"Unknown compile mode {compile_mode!r}")
    return _native.lib()
