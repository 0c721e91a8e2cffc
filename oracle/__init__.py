"""CPU oracle for the MoE grouped-GEMM hot path.  TEST INFRASTRUCTURE ONLY.

Everything in this package is a checker: a CPU restatement of the reference's arithmetic used by the
test-suite, by the smoke check and by the timed CPU-baseline leg of the benchmark.  The product package
never imports it, and the product has no CPU fallback.
"""
