"""Python entry to the CUDA kernels (ops.lib)."""
