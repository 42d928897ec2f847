"""CPU oracle for the fused VQ-attention path (test infrastructure, not product code).

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may
import this package; it is the checker, never the thing shipped or measured as the product.
"""
