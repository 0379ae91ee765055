"""CPU oracle for the SPLAT sparse-attention path (ACSR metadata, SDDMM, row softmax, SpMM).

TEST INFRASTRUCTURE ONLY.  Everything in this package is a CPU restatement of the reference
algorithm, used as the checker by the tests, by the smoke check and by the CPU-baseline leg of
the benchmark.  The shipped library never imports it and has no CPU fallback.

Pinning: the restatement is checked against fixtures produced by running the reference's own
Python code (``acsr_helpers.create_acsr``, ``r_sddmm.naive_block_mappings`` and the three Triton
kernels under the Triton interpreter, each on the sub-domain where that kernel is correct); the
fixtures and the script that generated them live in ``tests/golden``.
"""
