"""B200-native cuBLAS GEMM family behind the drop-in libcublas.so.12 / libcublasLt.so.12 / libnccl.so.2 C ABI.

The product is the three shared libraries under ``vulkanizer_b200/lib`` (sources in ``vulkanizer_b200/csrc``).
This Python package is only a ctypes binding to that C ABI for the test-suite and the benchmark: it loads the
libraries by absolute path, declares the prototypes, and refuses to work when a library is missing. It holds
no arithmetic and no fallback.
"""
from .capi import (  # noqa: F401
    LIB_DIR,
    BlasError,
    Cublas,
    CublasLt,
    NcclComm,
    nccl_library,
    build_libraries,
    cublas_library,
    cublaslt_library,
    declared_symbols,
)
