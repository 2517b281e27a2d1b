"""CPU oracle for the packed-KV hot path (test infrastructure, never shipped).

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this package.  The product (`residualquant_b200`) never does.
"""
