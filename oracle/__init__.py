"""TEST INFRASTRUCTURE ONLY - CPU restatement of the reference's decode path.

Nothing in the product package may import this directory.  It exists so that
tests, the smoke check and the benchmark's CPU-baseline leg have an independent
answer to compare the CUDA kernels with.
"""
