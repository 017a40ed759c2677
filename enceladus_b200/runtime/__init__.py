"""Launch path: `@jit` kernels, the kernel registry, interop with torch/NumPy and the autotuner."""
