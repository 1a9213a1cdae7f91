"""The reference's own CUDA operator in the GPU parity tests (test infrastructure).

The loader lives in ``oracle/reference_cuda.py``.  The comparisons with the
reference's CUDA operator are the strongest parity evidence there is, so a
missing module FAILS them (:func:`require`); only an explicit
``ATK_ALLOW_MISSING_REFERENCE=1`` in the environment turns the failure into a
skip (for a machine that has neither the reference checkout nor the prebuilt
module).
"""

from __future__ import annotations

import os

from oracle.reference_cuda import SO_PATH, available, module, reference_stage1, reference_topk  # noqa: F401


def require() -> None:
    """Call first in every test that compares with the reference's CUDA operator."""
    if available():
        return
    import pytest

    msg = (f"{SO_PATH} is missing: build it with `python oracle/build_ref.py --reference-root <reference checkout>` "
           "(or set ATK_ALLOW_MISSING_REFERENCE=1 to skip the comparisons with the reference's CUDA operator)")
    if os.environ.get("ATK_ALLOW_MISSING_REFERENCE") == "1":
        pytest.skip(msg)
    pytest.fail(msg)
