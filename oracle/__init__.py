"""TEST INFRASTRUCTURE ONLY: CPU checkers for the CUDA attention path.

Nothing in the shipped package imports this; only the test-suite, the smoke
check and the benchmark's CPU-baseline leg do.
"""
