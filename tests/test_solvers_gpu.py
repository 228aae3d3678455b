"""Triangular solves and batched LU / QR through the C ABI: cublasS/Dtrsm(+Batched), getrfBatched, getrsBatched, geqrfBatched.

The trsm cases restate k0zi/Vulkanizer's testTrsm (tests/cublas.cpp:193-261): every side / fill / transpose / diagonal
combination on a pointer-array batch, garbage in the triangle that must not be read, checked through the residual against
1e-4. The reference has no test of its batched LU and QR entry points (src/cublas/cublas.cpp:1336-1352, 1420-1431); they are
held here to LAPACK itself (scipy), whose conventions the reference's kernels state they follow (first largest pivot, 1-based
pivots, info = first zero pivot, dlarfg reflectors: src/linalg/shaders/lu_panel.comp:5-9, qr_panel.comp:5-8).
"""
import ctypes as C
import itertools

import numpy as np
import pytest
import scipy.linalg

from harness import DeviceBuffer
from vulkanizer_b200 import capi

L, U, NU, UN, LEFT, RIGHT = capi.FILL_LOWER, capi.FILL_UPPER, capi.DIAG_NON_UNIT, capi.DIAG_UNIT, capi.SIDE_LEFT, capi.SIDE_RIGHT
N, T = capi.OP_N, capi.OP_T


@pytest.fixture(scope="module")
def blas(cuda):
    handle = capi.Cublas()
    yield handle
    handle.destroy()


def pointer_array(cuda, buffers_and_strides, batch):
    ptrs = []
    for buf, stride_bytes in buffers_and_strides:
        ptrs += [buf.ptr + t * stride_bytes for t in range(batch)]
    return DeviceBuffer(cuda, np.array(ptrs, dtype=np.uint64))


def triangle_problem(rng, order, m, n, lda, ldb, batch, uplo, dtype):
    a = np.full((batch, order, lda), 1e6, dtype=dtype)          # [t][col][row]; the unused triangle holds garbage
    for t in range(batch):
        for c in range(order):
            for r in range(order):
                if r == c:
                    a[t, c, r] = 2.0 + 0.1 * r
                elif (r > c) == (uplo == L):
                    a[t, c, r] = rng.uniform(-0.25, 0.25)
    b = rng.uniform(-1, 1, size=(batch, n, ldb)).astype(dtype)
    return a, b


def op_of(a, order, uplo, trans, diag):
    """op(A) of one batch entry as a dense order x order matrix with the unused triangle zero."""
    stored = a[:, :order].T.astype(np.float64)                 # [row][col]
    tri = np.tril(stored, -1) if uplo == L else np.triu(stored, 1)
    tri = tri + (np.eye(order) if diag == UN else np.diag(np.diag(stored)))
    return tri.T if trans == T else tri


@pytest.mark.gpu
@pytest.mark.parametrize("side, uplo, trans, diag", list(itertools.product([LEFT, RIGHT], [L, U], [N, T], [NU, UN])))
def test_strsm_batched_every_combination(cuda, blas, side, uplo, trans, diag):
    m, n, batch, alpha = 7, 5, 3, 1.5
    order = m if side == LEFT else n
    lda, ldb = order + 1, m + 2
    rng = np.random.default_rng(77 + side * 8 + uplo * 4 + trans * 2 + diag)
    a, b = triangle_problem(rng, order, m, n, lda, ldb, batch, uplo, np.float32)
    dA, dB = DeviceBuffer(cuda, a.ravel()), DeviceBuffer(cuda, b.ravel())
    dP = pointer_array(cuda, [(dA, lda * order * 4), (dB, ldb * n * 4)], batch)
    al = C.c_float(alpha)
    status = blas.lib.cublasStrsmBatched(blas.handle, side, uplo, trans, diag, m, n, C.addressof(al), dP.ptr, lda, dP.ptr + 8 * batch, ldb, batch)
    assert status == capi.STATUS_SUCCESS
    x = dB.download().reshape(batch, n, ldb)
    for t in range(batch):
        opa, xm, bm = op_of(a[t], order, uplo, trans, diag), x[t, :, :m].T.astype(np.float64), b[t, :, :m].T.astype(np.float64)
        lhs = opa @ xm if side == LEFT else xm @ opa
        assert np.abs(lhs - alpha * bm).max() < 1e-4
        assert np.array_equal(x[t, :, m:], b[t, :, m:])        # the padding rows of B are not touched


@pytest.mark.gpu
@pytest.mark.parametrize("dtype, side, uplo, trans, diag, m, n", [
    (np.float32, LEFT, L, N, NU, 700, 300), (np.float32, LEFT, U, T, UN, 515, 70), (np.float32, RIGHT, U, N, NU, 200, 600),
    (np.float32, RIGHT, L, T, NU, 130, 333), (np.float64, LEFT, U, N, NU, 300, 40), (np.float64, RIGHT, L, N, UN, 64, 290)])
def test_trsm_single_large_blocked(cuda, blas, dtype, side, uplo, trans, diag, m, n):
    """One large system: diagonal blocks by the solve kernel, the rest by this repository's GEMM (orders above 256)."""
    order = m if side == LEFT else n
    lda, ldb, alpha = order + 3, m + 1, -0.75
    rng = np.random.default_rng(5)
    a, b = triangle_problem(rng, order, m, n, lda, ldb, 1, uplo, dtype)
    a[0][np.abs(a[0]) < 1e5] *= 4.0 / order                    # keep the system well conditioned at this size
    for r in range(order):
        a[0, r, r] = 2.0 + 0.1 * (r % 7)
    dA, dB = DeviceBuffer(cuda, a.ravel()), DeviceBuffer(cuda, b.ravel())
    al = (C.c_float if dtype == np.float32 else C.c_double)(alpha)
    fn = blas.lib.cublasStrsm_v2 if dtype == np.float32 else blas.lib.cublasDtrsm_v2
    assert fn(blas.handle, side, uplo, trans, diag, m, n, C.addressof(al), dA.ptr, lda, dB.ptr, ldb) == capi.STATUS_SUCCESS
    x = dB.download().reshape(n, ldb)[:, :m].T.astype(np.float64)
    opa, bm = op_of(a[0], order, uplo, trans, diag), b[0, :, :m].T.astype(np.float64)
    want = scipy.linalg.solve(opa, alpha * bm) if side == LEFT else scipy.linalg.solve(opa.T, alpha * bm.T).T
    tol = (2e-4 if dtype == np.float32 else 1e-11) * max(1.0, np.abs(want).max())
    assert np.abs(x - want).max() < tol


@pytest.mark.gpu
@pytest.mark.parametrize("dtype, n, nrhs, batch, trans", [(np.float32, 5, 3, 4, N), (np.float32, 33, 7, 3, T), (np.float64, 64, 2, 2, N),
                                                         (np.float32, 130, 5, 2, N), (np.float64, 260, 3, 1, T)])
def test_getrf_and_getrs_batched_against_lapack(cuda, blas, dtype, n, nrhs, batch, trans):
    es = np.dtype(dtype).itemsize
    lda, ldb = n + 2, n + 1
    rng = np.random.default_rng(n)
    a = rng.standard_normal((batch, n, lda)).astype(dtype)      # [t][col][row]
    b = rng.standard_normal((batch, nrhs, ldb)).astype(dtype)
    dA, dB = DeviceBuffer(cuda, a.ravel()), DeviceBuffer(cuda, b.ravel())
    dP = pointer_array(cuda, [(dA, lda * n * es), (dB, ldb * nrhs * es)], batch)
    dPiv, dInfo = DeviceBuffer(cuda, np.full(n * batch, -7, dtype=np.int32)), DeviceBuffer(cuda, np.full(batch, -7, dtype=np.int32))
    getrf = blas.lib.cublasSgetrfBatched if dtype == np.float32 else blas.lib.cublasDgetrfBatched
    getrs = blas.lib.cublasSgetrsBatched if dtype == np.float32 else blas.lib.cublasDgetrsBatched
    assert getrf(blas.handle, n, dP.ptr, lda, dPiv.ptr, dInfo.ptr, batch) == capi.STATUS_SUCCESS
    lu, piv, info = dA.download().reshape(batch, n, lda), dPiv.download().reshape(batch, n), dInfo.download()
    assert (info == 0).all()
    tol = 2e-4 if dtype == np.float32 else 1e-11
    for t in range(batch):
        want_lu, want_piv = scipy.linalg.lu_factor(a[t, :, :n].T.astype(np.float64))
        assert np.array_equal(piv[t] - 1, want_piv), "pivot rows (1-based here, 0-based in scipy)"
        assert np.abs(lu[t, :, :n].T - want_lu).max() < tol * max(1.0, np.abs(want_lu).max())
        assert np.array_equal(lu[t, :, n:], a[t, :, n:])        # padding rows untouched
    host_info = C.c_int(99)
    assert getrs(blas.handle, trans, n, nrhs, dP.ptr, lda, dPiv.ptr, dP.ptr + 8 * batch, ldb, C.byref(host_info), batch) == capi.STATUS_SUCCESS
    assert host_info.value == 0
    x = dB.download().reshape(batch, nrhs, ldb)
    for t in range(batch):
        am = a[t, :, :n].T.astype(np.float64)
        want = np.linalg.solve(am.T if trans == T else am, b[t, :, :n].T.astype(np.float64))
        assert np.abs(x[t, :, :n].T - want).max() < 50 * tol * max(1.0, np.abs(want).max())
    # invalid arguments are reported through the host integer
    assert getrs(blas.handle, trans, n, nrhs, dP.ptr, n - 1, dPiv.ptr, dP.ptr + 8 * batch, ldb, C.byref(host_info), batch) == capi.STATUS_INVALID_VALUE
    assert host_info.value == -5


@pytest.mark.gpu
def test_getrf_reports_the_first_zero_pivot_and_runs_without_pivoting(cuda, blas):
    n, batch = 4, 2
    a = np.zeros((batch, n, n), dtype=np.float32)
    a[0] = np.array([[2, 1, 0, 0], [4, 2, 0, 0], [0, 0, 1, 0], [0, 0, 0, 1]], dtype=np.float32).T   # column 1 becomes zero below row 0
    a[1] = (np.eye(n) * 3 + 0.1).astype(np.float32)
    dA = DeviceBuffer(cuda, a.ravel())
    dP = pointer_array(cuda, [(dA, n * n * 4)], batch)
    dPiv, dInfo = DeviceBuffer(cuda, np.zeros(n * batch, dtype=np.int32)), DeviceBuffer(cuda, np.zeros(batch, dtype=np.int32))
    assert blas.lib.cublasSgetrfBatched(blas.handle, n, dP.ptr, n, dPiv.ptr, dInfo.ptr, batch) == capi.STATUS_SUCCESS
    assert list(dInfo.download()) == [2, 0]
    dA2 = DeviceBuffer(cuda, a[1].ravel())
    dP2 = pointer_array(cuda, [(dA2, n * n * 4)], 1)
    assert blas.lib.cublasSgetrfBatched(blas.handle, n, dP2.ptr, n, None, dInfo.ptr, 1) == capi.STATUS_SUCCESS   # no pivoting
    lu = dA2.download().reshape(n, n).T.astype(np.float64)
    l, u = np.tril(lu, -1) + np.eye(n), np.triu(lu)
    assert np.abs(l @ u - a[1].T).max() < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("dtype, m, n, batch", [(np.float32, 7, 5, 3), (np.float32, 40, 40, 2), (np.float64, 90, 33, 2), (np.float32, 20, 50, 2),
                                                (np.float32, 300, 200, 1)])
def test_geqrf_batched_against_lapack(cuda, blas, dtype, m, n, batch):
    es = np.dtype(dtype).itemsize
    lda, k = m + 1, min(m, n)
    rng = np.random.default_rng(m * n)
    a = rng.standard_normal((batch, n, lda)).astype(dtype)
    dA, dTau = DeviceBuffer(cuda, a.ravel()), DeviceBuffer(cuda, np.zeros(k * batch, dtype=dtype))
    dP = pointer_array(cuda, [(dA, lda * n * es), (dTau, k * es)], batch)
    info = C.c_int(99)
    fn = blas.lib.cublasSgeqrfBatched if dtype == np.float32 else blas.lib.cublasDgeqrfBatched
    assert fn(blas.handle, m, n, dP.ptr, lda, dP.ptr + 8 * batch, C.byref(info), batch) == capi.STATUS_SUCCESS and info.value == 0
    qr, tau = dA.download().reshape(batch, n, lda), dTau.download().reshape(batch, k)
    tol = 3e-4 if dtype == np.float32 else 1e-11
    for t in range(batch):
        am = a[t, :, :m].T.astype(np.float64)
        want_qr, want_tau, _, _ = scipy.linalg.lapack.dgeqrf(am)
        assert np.abs(tau[t] - want_tau).max() < tol
        assert np.abs(qr[t, :, :m].T - want_qr).max() < tol * max(1.0, np.abs(want_qr).max())
    assert fn(blas.handle, m, n, dP.ptr, m - 1, dP.ptr + 8 * batch, C.byref(info), batch) == capi.STATUS_INVALID_VALUE and info.value == -4
