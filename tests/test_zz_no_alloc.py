"""The entry point for callers that may not allocate device memory: vkzbSgemmStaticScratch.

It runs the split-k fp32 kernel on a scratch array that is part of the library image instead of on memory a cuBLAS handle
allocated. The check: through the C ABI, its result equals what cublasSgemm_v2 (the existing entry point, on a handle) gives
for the same operands, within the tolerance the fp32 tests use (1e-5 * sqrt(k + 1), relative to max(1, |value|)), on two calls
in a row; the second call uses other operands and a different shape, so a counter or partial tile left over by the first
would show. A result too large for the built-in array must be refused and leave C as it was.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes as C
import math

import numpy as np
import pytest

from harness import DeviceBuffer, N, T
from oracle import pyoracle as orc
from vulkanizer_b200 import capi


def both_ways(torch, blas, ta, tb, m, n, k, alpha, beta, seed):
    rows_a, cols_a = (k, m) if ta == T else (m, k)
    rows_b, cols_b = (n, k) if tb == T else (k, n)
    lda, ldb, ldc = rows_a + 3, rows_b + 1, m + 2
    A, _ = orc.fill_lcg("f32", lda * cols_a, seed)
    B, _ = orc.fill_lcg("f32", ldb * cols_b, seed + 1)
    C0, _ = orc.fill_lcg("f32", ldc * n, seed + 2)
    dA, dB = DeviceBuffer(torch, A), DeviceBuffer(torch, B)
    d_handle, d_static = DeviceBuffer(torch, C0), DeviceBuffer(torch, C0)
    blas.sgemm(ta, tb, m, n, k, alpha, dA.ptr, lda, dB.ptr, ldb, beta, d_handle.ptr, ldc)
    a, b = C.c_float(alpha), C.c_float(beta)
    status = blas.lib.vkzbSgemmStaticScratch(None, ta, tb, m, n, k, C.addressof(a), dA.ptr, lda, dB.ptr, ldb, C.addressof(b), d_static.ptr, ldc)
    assert status == capi.STATUS_SUCCESS
    want, got = d_handle.download(), d_static.download()  # download() also checks the guard bands around C
    tol = 1e-5 * np.maximum(1.0, np.abs(want)) * math.sqrt(k + 1)
    assert (np.abs(got - want) <= tol).all(), f"largest difference {np.abs(got - want).max()}"
    assert not np.array_equal(got, C0)


@pytest.mark.gpu
def test_static_scratch_sgemm_matches_the_handle_entry_point_twice_in_a_row(cuda):
    blas = capi.Cublas()
    try:
        both_ways(cuda, blas, N, N, 512, 512, 512, 1.0, 0.5, 11)       # the benchmark's fp32 shape: four k slices
        both_ways(cuda, blas, T, N, 200, 130, 1000, -0.75, 2.0, 21)    # other operands, ragged tiles, another slice count
    finally:
        blas.destroy()


@pytest.mark.gpu
def test_static_scratch_sgemm_refuses_what_does_not_fit(cuda):
    lib = capi.cublas_library()
    m = n = 2048  # 1024 tiles of 64 x 64: four times the built-in array
    A, _ = orc.fill_lcg("f32", m * 8, 1)
    C0 = np.full(16, 3.0, dtype=np.float32)
    dA, dC = DeviceBuffer(cuda, A), DeviceBuffer(cuda, C0)
    a, b = C.c_float(1.0), C.c_float(0.0)
    status = lib.vkzbSgemmStaticScratch(None, N, N, m, n, 8, C.addressof(a), dA.ptr, m, dA.ptr, 8, C.addressof(b), dC.ptr, m)
    assert status == capi.STATUS_INVALID_VALUE
    assert np.array_equal(dC.download(), C0)
    assert lib.vkzbSgemmStaticScratch(None, N, N, 64, 64, 0, C.addressof(a), dA.ptr, 64, dA.ptr, 1, C.addressof(b), dC.ptr, 64) == capi.STATUS_NOT_SUPPORTED
    assert lib.vkzbSgemmStaticScratch(None, N, N, 64, 64, 64, None, dA.ptr, 64, dA.ptr, 64, C.addressof(b), dC.ptr, 64) == capi.STATUS_INVALID_VALUE
