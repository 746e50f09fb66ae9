"""CPU oracle for the KV-placement hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; it exists so the CUDA path can be checked bit for bit against a
restatement of the reference algorithm.  Only the test-suite, the smoke check
and the CPU-baseline leg of the benchmark may import it.

Pinning: every function here is checked against outputs produced by running
the unmodified reference Python modules (fixtures under ``tests/golden``,
written by ``tests/golden/make_golden.py``).  The reference ships no tests or
golden vectors of its own.
"""
