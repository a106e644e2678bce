"""CPU oracle for the paged-attention decode path.

TEST INFRASTRUCTURE ONLY. Nothing in the shipped package imports this directory:
only the test-suite, the repository smoke check and the benchmark's CPU-baseline
leg may call it, and only as the checker / the timed CPU baseline, never as the
product path.

Parity status: PINNED. Every function here is checked against outputs of the
reference's own CPU implementation (``tests/paged_attention_reference.py``,
``tests/fp64_reference.py``, ``tests/decoder_cpu_reference.py`` of the reference
project), captured as fixtures under ``tests/golden/`` by
``tests/golden/make_golden.py``, and against the known-answer vectors that the
reference's tests carry (``tests/fused_norm_midpoint_smoke.py:19-35``,
``tests/decoder_cpu_reference_test.py:66-68``, ``tests/attention_plan_smoke.py:29-38``,
``tests/paged_slots_device_smoke.py:16-37``); the grammar-bitmask rule and the rank-ordered sum are
pinned by outputs of the reference's own ``ref_apply_bitmask`` / ``_canonical_rank_sum``
(``tests/golden/after_attention.npz``).  Unpinned corners (no reference test
exercises them): ``weight_offset != 0`` in the RMS norms; row code 5 of
``device_metadata_status`` (the reference's validating kernel is not in its tree; codes
1-4, 6 and 7 are the ones ``tests/paged_device_metadata_smoke.py:130-150`` expects).
"""
from .paged_oracle import *  # noqa: F401,F403
