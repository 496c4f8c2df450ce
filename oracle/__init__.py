"""CPU oracle for the Llama-block op path. TEST INFRASTRUCTURE ONLY.

Nothing under this package is part of the product: the shipped ops live in
``custom_cuda_kernals_b200`` and never import from here.  Only the test-suite,
``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of
``bench.py`` may use it, and only as the checker.

The functions restate, in independent code, the op chains of the reference
project's PyTorch baselines (``baselines/*.py`` in
BhargavKumarNath/custom_cuda_kernals); each function's docstring cites the
reference lines it follows because the order of casts decides the rounding.

Parity pin: the restatement is compared against the reference's own
``baselines`` functions, imported from a checkout of the reference, by
``tests/golden/make_golden.py``; that script also writes the golden vectors
under ``tests/golden/`` which ``tests/test_oracle_golden.py`` replays on any
machine.  Variants the reference has no baseline for (per-token FP8 scales,
the FP8 GEMM) are restated from the same chain and are marked "unpinned by the
reference" in their docstrings.
"""

from . import cases, ops, workloads  # noqa: F401
