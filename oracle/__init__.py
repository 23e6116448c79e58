"""CPU oracle for the GGUF quantized-matmul path: test infrastructure only.

Only the tests, the smoke check and the benchmark's CPU-baseline leg may import this package.
"""
