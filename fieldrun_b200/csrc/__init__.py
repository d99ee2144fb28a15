"""CUDA sources for sm_100a, their build and their Python bindings."""
