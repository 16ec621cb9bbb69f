"""CPU oracle for the causal-attention path (test infrastructure, not product code).

Only the tests, the smoke check and the CPU-baseline leg of the benchmark may
import this package.
"""
