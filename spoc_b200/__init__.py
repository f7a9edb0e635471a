"""spoc_b200 — B200 (sm_100a) backend for Sarek's dense-GEMM and fused-map path.

The product is ``libsarek_b200.so`` (CUDA kernels behind a C ABI, see
``include/sb200.h``).  ``plugin`` mirrors the reference's plugin interface on
top of it; ``sarek_ir`` builds the IR text the backend consumes; ``build``
compiles the library in-tree.
"""
from . import _lib  # noqa: F401
from .plugin import (Backend, BackendError, UnsupportedConstruct, Dims, dims1d, dims2d, Vector, run_vectors,  # noqa: F401
                     RSA_Buffer, RSA_Int32, RSA_Int64, RSA_Float32, RSA_Float64)

__all__ = ["Backend", "BackendError", "UnsupportedConstruct", "Dims", "dims1d", "dims2d", "Vector", "run_vectors",
           "RSA_Buffer", "RSA_Int32", "RSA_Int64", "RSA_Float32", "RSA_Float64"]
