"""Python side of the CUDA kernels: ``build`` compiles and loads them, ``ops`` wraps them."""
