"""TEST INFRASTRUCTURE: CPU oracle for the SORT task.

Nothing under this directory is part of the product.  Only the test-suite, the
smoke check and the benchmark's CPU-baseline / reference arm may import it.

Two restatements of the reference's CPU arithmetic live here:

* ``thrust_oracle`` - the reference's CPU/OpenMP variant call for call
  (``src/cupynumeric/sort/sort_cpu.inl:52-85``) through the same Thrust
  ``host`` / ``omp`` back-ends, compiled from ``oracle_thrust.cpp``.
* ``np_oracle`` - NumPy's stable sort, which is the oracle the reference's own
  integration tests use (``tests/integration/test_sort.py:85-102``,
  ``tests/integration/test_argsort.py:132-163``).

Both are pinned against the golden vectors of the reference's C++ tests
(``tests/cpp/integration/test_sort.cc``, ``test_argsort.cc``) by
``tests/test_oracle.py``.  NaN placement is *parity unpinned*: the reference
has no test with NaN input; the contract used here is NumPy's NaN-last order.
"""
from .np_oracle import np_sort, np_argsort, np_task_sort, complex_lex_argsort  # noqa: F401
from .thrust_oracle import thrust_task_sort, num_threads, set_num_threads, build as build_thrust_oracle  # noqa: F401
