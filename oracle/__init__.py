"""CPU oracle of the sparse graph-attention path.  TEST INFRASTRUCTURE ONLY.

Nothing under this package is part of the product: only ``tests/``, ``__graft_entry__.smoke()`` and
the CPU-baseline / reference legs of ``bench.py`` may import it, and only as the checker or the
timed CPU baseline.  The product (``torchgt_b200``) never imports it and has no CPU fallback.

Parity status: the reference project ships no tests and no golden vectors, so the restatements
here are pinned against the reference itself — its own ``CoreAttention.sparse_attention_bias``,
``_SeqAllToAll`` index maps and edge-index helpers were imported and run on seeded inputs, and the
results are committed under ``tests/golden/`` together with the script that produced them
(``tests/golden/make_golden.py``).
"""
