"""Functional API over the CUDA kernels; names follow the reference's ``engine/kernels``."""
