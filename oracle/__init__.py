"""CPU restatement of the reference's attention hot path.  TEST INFRASTRUCTURE ONLY.

Nothing under this directory is part of the product: only the tests, the smoke check and the
CPU-baseline leg of the benchmark may import it, and only as the checker.  Each function cites
the file and lines of MindIE-SD it restates.  Parity is pinned: `tests/test_oracle_golden.py`
compares every function here with vectors produced by running the reference's own Python code
(see `tests/golden/make_golden.py`).
"""
