"""CPU oracle for the batch-1 FP8 decode path -- TEST INFRASTRUCTURE ONLY.

This package restates, in plain PyTorch on the CPU, the reference's per-operator
``golden_forward`` methods (tilert/models/deepseek_v3_2/ops/*.py) and adds the three
pieces the reference never states in Python: the layer/model composition, the
lightning-indexer scoring formula and the greedy arg-max over the vocabulary.

Nothing in the shipped package may import this module.  Only the test-suite, the
smoke check and the benchmark's CPU-baseline leg use it, and only as the checker.

Parity pin: the reference ships no tests and no golden vectors for this path, so the
restatement is pinned against the reference's own ``golden_forward`` code, imported
and run on seeded inputs by ``oracle/pin_reference.py``; the outputs of that run are
committed under ``tests/golden/`` and re-checked by the CPU test tier.  The indexer
scoring formula and the model composition have no reference counterpart to pin
against ("parity unpinned" for those two pieces).
"""

from . import model, ops, quant  # noqa: F401
