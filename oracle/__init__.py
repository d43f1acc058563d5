"""CPU oracle for the GEMM / attention-forward hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product (``warpir_b200``) may import this package: it is the
checker used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.
"""
