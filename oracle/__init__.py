"""CPU oracle: the checker for the CUDA path. Only tests, the smoke check and the
bench's CPU-baseline legs import this package."""
