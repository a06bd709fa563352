"""CPU oracle for the LatentMoE feed-forward path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this directory.  The only callers are
the test-suite, the smoke check and the CPU-baseline / reference legs of the
benchmark, and there it is always the checker, never the thing being measured
as the product.

Parity status: PINNED.  The reference ships no tests or golden vectors for
this layer, so the restatement in ``latent_moe_ref.py`` is pinned against the
reference module itself (``models/moe.py: LatentMoELayer``), executed on CPU
with its two device-only entry points (``models/moe_triton.py:36-78`` and
``200-242``) replaced by equivalent torch code (``ref_shim.py``).  The frozen
outputs of that run live under ``tests/golden`` next to the script that made
them.  The FP8 fake-quantisation model (``fp8_model.py``) follows a
third-party dependency that is not vendored by the reference (torchao,
``requirements.txt``: ``torchao>=0.5.0``); that part is "parity unpinned".
"""
