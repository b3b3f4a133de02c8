"""CUDA sources of the kernels, their build, and the Python face of each
entry point (``ops``)."""
