"""CPU restatement of the reference algorithms (t-head/pla) for the hot path.

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this; only
``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / reference
legs of ``bench.py`` may use it, and only as the checker or the timed CPU arm.

Every function cites the reference file:line it restates. The restatements are
pinned against outputs of the reference's own PyTorch oracles, generated in a
container that has the reference tree by ``tests/golden/make_golden.py`` and
committed under ``tests/golden/``.
"""
