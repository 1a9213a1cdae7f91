"""CPU oracle for the bucketed approximate top-k path (test infrastructure only).

Nothing in the product package imports this module.  It is used by ``tests/``, by
the smoke check and by the CPU-baseline / reference legs of ``bench.py``.
"""
