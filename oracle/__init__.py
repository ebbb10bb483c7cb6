"""CPU oracle for the PCVR inference hot path — TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Everything in this package restates, in plain numpy / fp32 torch on the CPU, what the
reference project's torch path computes for the operators and the OneTrans forward that the
CUDA library accelerates.  Each function cites the reference file:line it follows, and the
package is pinned against outputs of the reference itself (``tests/golden/*.npz``, written by
``tests/golden/make_golden.py``).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / ``--impl reference`` legs
of ``bench.py`` may import this package, and only as the checker or the timed CPU baseline.
Nothing under ``taac_2026_b200/`` imports it; the product path has no CPU fallback.
"""
