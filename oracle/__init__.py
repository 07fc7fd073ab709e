"""CPU oracle (checker) for the CUDA kernels.  Test infrastructure, not product code."""
