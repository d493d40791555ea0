"""CPU checker for the CUDA kernels -- test infrastructure, never imported by the product."""
