"""Python side of the CUDA kernels: library loading, launch wrappers, dispatch."""
