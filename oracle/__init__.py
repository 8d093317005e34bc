"""CPU checker for the CUDA path.  Test infrastructure: only ``tests/``, the smoke
check and the CPU-baseline legs of ``bench.py`` may import this package."""
