"""CPU oracle for the GPT training-step path. TEST INFRASTRUCTURE ONLY.

Everything under this package is a NumPy restatement of the reference's CPU
algorithm for one function of the path, each citing the reference file:line
it follows. It exists to check the CUDA library, never to compute for it:
only the test suite, the smoke check and the benchmark's CPU-baseline /
reference arm may import it. The product package must not.

Parity status: PINNED. The reference has no golden vectors of its own, so the
oracle is pinned by running the unmodified reference (NumPy CPU path) on seeded
inputs; the outputs are committed under tests/golden/ together with the script
that produced them, and tests/test_oracle_golden.py checks every oracle
function against those files.
"""
