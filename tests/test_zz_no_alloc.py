"""The entry point for callers that may not allocate device memory: vkzbSgemmStaticScratch.

Who that is: a server that handed all device memory to its own pool at start-up, or code inside a latency-critical phase where
cudaMalloc's device-wide synchronisation is not acceptable. A cuBLAS handle of this library allocates its split-k scratch memory
at the first call that splits; this entry point instead runs the split-k fp32 kernel on a scratch array that is part of the
library image, so no call of it ever allocates.

The checks, all through the C ABI:
  * its result equals what cublasSgemm_v2 (the existing entry point, on a handle) gives for the same operands, within the
    tolerance the fp32 tests use (1e-5 * sqrt(k + 1), relative to max(1, |value|)), on two calls in a row; the second call uses
    other operands and another shape, so a counter or partial tile left over by the first would show;
  * both results are also held to the fp64 oracle (the handle path runs the same kernel, so agreeing with it alone would let a
    bug in that kernel through);
  * the largest result the built-in array takes (1024 x 1024), a k too short to split, and a call on a created stream;
  * the free device memory reported by the driver is the same before and after a call: nothing was allocated;
  * a result too large for the array is refused and C stays as it was.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes as C
import math

import numpy as np
import pytest

from harness import DeviceBuffer, N, T
from oracle import pyoracle as orc
from vulkanizer_b200 import capi


def static_sgemm(lib, stream, ta, tb, m, n, k, alpha, dA, lda, dB, ldb, beta, dC, ldc):
    a, b = C.c_float(alpha), C.c_float(beta)
    return lib.vkzbSgemmStaticScratch(stream, ta, tb, m, n, k, C.addressof(a), dA.ptr, lda, dB.ptr, ldb, C.addressof(b), dC.ptr, ldc)


def both_ways(torch, blas, ta, tb, m, n, k, alpha, beta, seed, stream=None):
    rows_a, cols_a = (k, m) if ta == T else (m, k)
    rows_b, cols_b = (n, k) if tb == T else (k, n)
    lda, ldb, ldc = rows_a + 3, rows_b + 1, m + 2
    A, _ = orc.fill_lcg("f32", lda * cols_a, seed)
    B, _ = orc.fill_lcg("f32", ldb * cols_b, seed + 1)
    C0, _ = orc.fill_lcg("f32", ldc * n, seed + 2)
    oracle, _ = orc.gemm_fp64(ta == T, tb == T, m, n, k, 1, alpha, A, "f32", lda, 0, B, "f32", ldb, 0, beta, C0, "f32", ldc, 0)
    dA, dB = DeviceBuffer(torch, A), DeviceBuffer(torch, B)
    d_handle, d_static = DeviceBuffer(torch, C0), DeviceBuffer(torch, C0)
    blas.sgemm(ta, tb, m, n, k, alpha, dA.ptr, lda, dB.ptr, ldb, beta, d_handle.ptr, ldc)
    torch.cuda.synchronize()
    status = static_sgemm(blas.lib, stream, ta, tb, m, n, k, alpha, dA, lda, dB, ldb, beta, d_static, ldc)
    assert status == capi.STATUS_SUCCESS
    want, got = d_handle.download(), d_static.download()  # download() synchronises and checks the guard bands around C
    tol = 1e-5 * np.maximum(1.0, np.abs(oracle)) * math.sqrt(k + 1)
    assert (np.abs(got - want) <= tol).all(), f"against the handle entry point: largest difference {np.abs(got - want).max()}"
    assert (np.abs(got - oracle) <= tol).all(), f"against the fp64 oracle: largest difference {np.abs(got - oracle).max()}"
    assert (np.abs(want - oracle) <= tol).all()
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
def test_static_scratch_sgemm_at_its_limits(cuda):
    blas = capi.Cublas()
    stream = cuda.cuda.Stream()
    try:
        both_ways(cuda, blas, N, T, 1024, 1024, 64, 1.0, 0.0, 31)     # 256 tiles: all the built-in array holds, one k slice
        both_ways(cuda, blas, T, T, 96, 70, 8, 2.0, -1.0, 41)         # k too short to cut
        cuda.cuda.synchronize()
        both_ways(cuda, blas, N, N, 300, 200, 700, 0.5, 0.25, 51, stream=stream.cuda_stream)   # on a created stream
        stream.synchronize()
    finally:
        blas.destroy()


@pytest.mark.gpu
def test_static_scratch_sgemm_allocates_nothing(cuda):
    lib = capi.cublas_library()
    m = n = k = 256
    A, _ = orc.fill_lcg("f32", m * k, 1)
    dA, dB, dC = DeviceBuffer(cuda, A), DeviceBuffer(cuda, A), DeviceBuffer(cuda, np.zeros(m * n, dtype=np.float32))
    assert static_sgemm(lib, None, N, N, m, n, k, 1.0, dA, m, dB, k, 0.0, dC, m) == capi.STATUS_SUCCESS   # set-up call: loads the module
    cuda.cuda.synchronize()
    free_before, _ = cuda.cuda.mem_get_info()
    for _ in range(3):
        assert static_sgemm(lib, None, N, N, m, n, k, 1.0, dA, m, dB, k, 0.0, dC, m) == capi.STATUS_SUCCESS
    cuda.cuda.synchronize()
    free_after, _ = cuda.cuda.mem_get_info()
    assert free_after == free_before, f"free device memory changed by {free_before - free_after} bytes across the calls"


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
