"""CUDA sources of the library, their build driver and their Python faces."""
