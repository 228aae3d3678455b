"""Behaviour of the C ABI beyond the case table: status codes, pointer modes, stream capture, int8, cuBLASLt, Sgemv, Dgemm.

Expectations follow k0zi/Vulkanizer: validation and early outs src/cublas/cublas.cpp:698-710; `_64` forms :1161-1209; Sgemv
:1143-1159 and tests/cublas.cpp:345-392; cuBLASLt tests/cublas.cpp:395-488 (D may differ from C, C stays untouched, D is rounded
once before bias / activation); f64 tests/cublas.cpp:265-340; 4 KiB-aliased leading dimensions checked on a sample of C,
tests/cublas.cpp:550-585. int8 has no counterpart in the reference: the expectation is exact integer arithmetic.
"""
import ctypes as C
import math

import numpy as np
import pytest

from harness import CUDA_TYPE, ELEM, DeviceBuffer, N, T
from oracle import pyoracle as orc
from vulkanizer_b200 import capi


@pytest.fixture(scope="module")
def blas(cuda):
    b = capi.Cublas()
    yield b
    b.destroy()


@pytest.fixture(scope="module")
def lt(cuda):
    h = capi.CublasLt()
    yield h
    h.destroy()


# ---- status codes ------------------------------------------------------------------------------------------------

@pytest.mark.gpu
def test_validation_and_early_outs(cuda, blas):
    A, _ = orc.fill_lcg("f32", 64, 1)
    d = DeviceBuffer(cuda, A)
    p = d.ptr
    S = capi
    assert blas.sgemm(N, N, -1, 2, 2, 1.0, p, 2, p, 2, 0.0, p, 2, check=False) == S.STATUS_INVALID_VALUE      # negative size
    assert blas.sgemm(N, N, 4, 2, 2, 1.0, p, 3, p, 2, 0.0, p, 4, check=False) == S.STATUS_INVALID_VALUE       # lda < rows of A
    assert blas.sgemm(T, N, 4, 2, 2, 1.0, p, 1, p, 2, 0.0, p, 4, check=False) == S.STATUS_INVALID_VALUE       # op(A) = T: lda < k
    assert blas.sgemm(N, N, 4, 2, 2, 1.0, p, 4, p, 2, 0.0, p, 3, check=False) == S.STATUS_INVALID_VALUE       # ldc < m
    assert blas.sgemm(7, N, 4, 2, 2, 1.0, p, 4, p, 2, 0.0, p, 4, check=False) == S.STATUS_INVALID_VALUE       # bad operation
    before = blas.launch_count()
    assert blas.sgemm(N, N, 0, 2, 2, 1.0, p, 1, p, 2, 0.0, p, 1, check=False) == S.STATUS_SUCCESS             # m = 0: nothing to do
    assert blas.sgemm(N, N, 2, 0, 2, 1.0, p, 2, p, 2, 0.0, p, 2, check=False) == S.STATUS_SUCCESS
    assert blas.launch_count() == before and blas.last_path() == S.PATH_NONE
    # null alpha
    lib = blas.lib
    assert lib.cublasSgemm_v2(blas.handle, N, N, 2, 2, 2, None, p, 2, p, 2, None, p, 2) == S.STATUS_INVALID_VALUE
    # unsupported type combinations
    assert blas.gemm_ex(N, N, 2, 2, 2, 1.0, p, S.CUDA_R_8I, 4, p, S.CUDA_R_8I, 4, 0.0, p, S.CUDA_R_32F, 4, S.COMPUTE_32F, check=False) == S.STATUS_NOT_SUPPORTED
    assert blas.gemm_ex(N, N, 2, 2, 2, 1.0, p, 4, 4, p, 4, 4, 0.0, p, 4, 4, S.COMPUTE_32F, check=False) == S.STATUS_NOT_SUPPORTED  # complex
    assert lib.cublasSgemm_v2_64(blas.handle, N, N, 1 << 32, 1, 1, None, p, 1 << 32, p, 1, None, p, 1 << 32) == S.STATUS_NOT_SUPPORTED
    assert d.download() is not None  # guard bands intact


@pytest.mark.gpu
def test_k_zero_and_beta_zero_semantics(cuda, blas):
    """k = 0 scales C by beta (tests/cublas.cpp:662); beta = 0 must not read C, so NaNs in C do not propagate."""
    m, n, k = 70, 33, 40
    A, av = orc.fill_lcg("f16", m * k, 1)
    B, bv = orc.fill_lcg("f16", k * n, 2)
    Cn = np.full(m * n, np.nan, dtype=np.float32)
    dA, dB, dC = DeviceBuffer(cuda, A), DeviceBuffer(cuda, B), DeviceBuffer(cuda, Cn)
    blas.gemm_ex(T, N, m, n, k, 1.0, dA.ptr, capi.CUDA_R_16F, k, dB.ptr, capi.CUDA_R_16F, k, 0.0, dC.ptr, capi.CUDA_R_32F, m)
    got = dC.download()
    want = av.reshape(m, k).astype(np.float64) @ bv.reshape(n, k).astype(np.float64).T
    assert np.isfinite(got).all() and np.allclose(got.reshape(n, m).T, want, atol=1e-4)


# ---- pointer modes and stream capture ------------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(256, 136, 192, "f16"), (200, 130, 100, "f32"), (300, 1, 257, "f16")])
def test_device_pointer_mode_inside_stream_capture(cuda, shape):
    """alpha and beta live on the device and the call is captured into a CUDA graph: nothing may synchronise or copy back
    (the reference copies each scalar to the host with a blocking call, cublas.cpp:241-243, and so cannot be captured)."""
    torch = cuda
    m, n, k, kind = shape
    A, _ = orc.fill_lcg(kind, m * k, 1)
    B, _ = orc.fill_lcg(kind, k * n, 2)
    Cm, _ = orc.fill_lcg("f32", m * n, 3)
    want, want_abs = orc.gemm_fp64(True, False, m, n, k, 1, 0.75, A, kind, k, 0, B, kind, k, 0, -1.5, Cm, "f32", m, 0)
    dA, dB, dC = DeviceBuffer(torch, A), DeviceBuffer(torch, B), DeviceBuffer(torch, Cm)
    scalars = torch.tensor([0.75, -1.5], dtype=torch.float32, device="cuda")
    b = capi.Cublas()
    b.set_pointer_mode(capi.POINTER_MODE_DEVICE)
    stream = torch.cuda.Stream()
    b.set_stream(stream.cuda_stream)
    t = CUDA_TYPE[kind]
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            b.gemm_ex(T, N, m, n, k, scalars.data_ptr(), dA.ptr, t, k, dB.ptr, t, k, scalars.data_ptr() + 4, dC.ptr, capi.CUDA_R_32F, m,
                      device_scalars=True)
    torch.cuda.synchronize()
    assert np.array_equal(dC.download(), Cm), "capturing must not run the kernel"
    graph.replay()
    torch.cuda.synchronize()
    got = dC.download()
    tol = 1e-5 * np.maximum(1, np.abs(want)) * math.sqrt(k + 1)
    assert (np.abs(got - want) <= tol).all()
    b.destroy()


# ---- int8 -> int32 (bit exact) ---------------------------------------------------------------------------------------

S8_CASES = [
    # ta, tb, m, n, k, lda pad, alpha, beta, batch
    ("tn aligned tensor cores", T, N, 256, 192, 512, 0, 1, 0, 1),
    ("tn ragged edges", T, N, 200, 137, 400, 0, 1, 0, 1),
    ("tn k tail and beta", T, N, 130, 72, 1000, 0, 3, -2, 1),
    ("tn batched", T, N, 128, 96, 256, 0, 1, 0, 5),
    ("tn long k", T, N, 64, 48, 11008, 0, 1, 0, 1),
    ("nn aligned", N, N, 256, 128, 256, 0, 1, 0, 1),
    ("nt aligned", N, T, 144, 160, 192, 0, 2, 1, 1),
    ("tt aligned", T, T, 160, 144, 320, 0, 1, 0, 1),
    ("tn unaligned ld (generic kernel)", T, N, 70, 33, 129, 3, 1, 1, 1),
    ("gemv int8", T, N, 300, 1, 512, 0, 1, 0, 1),
    # few tiles and a long k: the tensor-core kernel splits along k and sums the parts through scratch memory
    ("tn split along k, tile pairs", T, N, 512, 512, 4096, 0, 1, 0, 1),
    ("nn split along k with beta", N, N, 256, 128, 4096, 0, 2, -1, 1),
    ("tn split along k, ragged and batched", T, N, 200, 96, 2048, 0, 1, 1, 3),
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", S8_CASES, ids=lambda c: c[0])
def test_int8_gemm_is_bit_exact(cuda, blas, case):
    from vulkanizer_b200 import synth
    name, ta, tb, m, n, k, pad, alpha, beta, batch = case
    rows_a, cols_a = (k, m) if ta == T else (m, k)
    rows_b, cols_b = (n, k) if tb == T else (k, n)
    lda, ldb, ldc = rows_a + pad, rows_b + pad, m + (2 if pad else 0)
    sA, sB, sC = lda * cols_a, ldb * cols_b, ldc * n
    A = synth.int8_uniform(2, sA * batch)
    B = synth.int8_uniform(2, sB * batch, first=sA * batch)
    C0 = (synth.int8_uniform(9, sC * batch).astype(np.int32)) * 1000
    want = orc.gemm_s8(ta == T, tb == T, m, n, k, batch, alpha, A, lda, sA, B, ldb, sB, beta, C0.copy(), ldc, sC)
    dA, dB, dC = DeviceBuffer(cuda, A), DeviceBuffer(cuda, B), DeviceBuffer(cuda, C0)
    blas.gemm_strided_batched_ex(ta, tb, m, n, k, alpha, dA.ptr, capi.CUDA_R_8I, lda, sA, dB.ptr, capi.CUDA_R_8I, ldb, sB, beta, dC.ptr,
                                 capi.CUDA_R_32I, ldc, sC, batch, capi.COMPUTE_32I)
    got = dC.download()
    assert np.array_equal(got, want), f"{name}: {int((got != want).sum())} of {got.size} differ"
    if "tensor cores" in name or "aligned" in name and "unaligned" not in name:
        assert blas.last_path() == capi.PATH_UMMA
    assert blas.device_status() == 0


# ---- cuBLASLt ----------------------------------------------------------------------------------------------------------

LT_CASES = [
    ("lt TN bias", T, N, 70, 33, 40, 1, "f32", capi.LT_EPILOGUE_BIAS, 1.0, 0.0),
    ("lt NN relu bias beta", N, N, 50, 20, 64, 1, "f32", capi.LT_EPILOGUE_RELU_BIAS, 0.5, 1.5),
    ("lt TN gelu bias f16", T, N, 64, 48, 32, 1, "f16", capi.LT_EPILOGUE_GELU_BIAS, 1.0, 0.0),
    ("lt NT default batched", N, T, 30, 17, 25, 3, "f32", capi.LT_EPILOGUE_DEFAULT, 1.0, -1.0),
    ("lt TN gelu bf16 tensor cores", T, N, 256, 136, 128, 2, "bf16", capi.LT_EPILOGUE_GELU, 1.0, 0.5),
    ("lt TN relu bias f16 tensor cores", T, N, 384, 264, 192, 1, "f16", capi.LT_EPILOGUE_RELU_BIAS, 0.5, 0.0),
    ("lt TN default f16 -> D != C", T, N, 256, 128, 64, 1, "f16", capi.LT_EPILOGUE_DEFAULT, 1.0, 2.0),
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", LT_CASES, ids=lambda c: c[0])
def test_lt_matmul_fused_epilogue(cuda, lt, case):
    name, ta, tb, m, n, k, batch, kind, epilogue, alpha, beta = case
    rows_a, cols_a = (k, m) if ta == T else (m, k)
    rows_b, cols_b = (n, k) if tb == T else (k, n)
    sA, sB, sC = rows_a * cols_a, rows_b * cols_b, m * n
    A, _ = orc.fill_lcg(kind, sA * batch, 31)
    B, _ = orc.fill_lcg(kind, sB * batch, 32)
    Cm, _ = orc.fill_lcg(kind, sC * batch, 33)
    D0, _ = orc.fill_lcg(kind, sC * batch, 34)
    bias, _ = orc.fill_lcg(kind, m, 35)
    bits = (1 if epilogue & capi.LT_EPILOGUE_BIAS else 0) | (2 if (epilogue & ~4) == capi.LT_EPILOGUE_RELU else 0) | \
           (4 if (epilogue & ~4) == capi.LT_EPILOGUE_GELU else 0)
    want = orc.lt_fp64(ta == T, tb == T, m, n, k, batch, alpha, A, B, beta, Cm, bias, kind, bits)
    dA, dB, dC, dD, dBias = (DeviceBuffer(cuda, x) for x in (A, B, Cm, D0, bias))
    t = CUDA_TYPE[kind]
    lt.matmul(ta, tb, m, n, k, alpha, dA.ptr, t, rows_a, dB.ptr, t, rows_b, beta, dC.ptr, t, m, dD.ptr, t, m, epilogue=epilogue,
              bias=dBias.ptr, batch=batch, stride_a=sA, stride_b=sB, stride_c=sC, stride_d=sC)
    got = orc.to_float(dD.download(), kind)
    rel = 1e-5 if kind == "f32" else 4e-3 if kind == "f16" else 1.6e-2
    tol = rel * np.maximum(1.0, np.abs(want)) * math.sqrt(k)
    bad = ~(np.abs(got - want) <= tol)
    assert not bad.any(), f"{name}: {int(bad.sum())} wrong, first got {got[np.argmax(bad)]} want {want[np.argmax(bad)]}"
    assert np.array_equal(dC.download(), Cm), "C is only read"
    if "tensor cores" in name:
        assert lt.last_path() == capi.PATH_UMMA


@pytest.mark.gpu
def test_lt_refuses_what_it_does_not_serve(cuda, lt):
    A, _ = orc.fill_lcg("f32", 64 * 64, 1)
    d = DeviceBuffer(cuda, A)
    args = (N, N, 8, 8, 8, 1.0, d.ptr, capi.CUDA_R_32F, 8, d.ptr, capi.CUDA_R_32F, 8, 0.0, d.ptr, capi.CUDA_R_32F, 8, d.ptr, capi.CUDA_R_32F, 8)
    assert lt.matmul(*args, epilogue=128 | 2, check=False) == capi.STATUS_INVALID_VALUE   # RELU_AUX without an auxiliary pointer
    assert lt.matmul(*args, epilogue=128 | 2 | 1, check=False) == capi.STATUS_NOT_SUPPORTED  # not one of NVIDIA's epilogue numbers
    assert lt.matmul(*args, order=(0, 0, 1, 0), check=False) == capi.STATUS_NOT_SUPPORTED  # C and D in different orders
    assert lt.matmul(*args, order=1, epilogue=capi.LT_EPILOGUE_GELU_AUX, aux=d.ptr, aux_ld=8, check=False) == capi.STATUS_NOT_SUPPORTED  # aux with row-order D
    assert lt.matmul(*args, epilogue=capi.LT_EPILOGUE_BIAS, bias=0, check=False) == capi.STATUS_INVALID_VALUE  # bias epilogue without a pointer
    assert lt.matmul(*args, check=False) == capi.STATUS_SUCCESS


@pytest.mark.gpu
def test_cublas_handle_is_a_valid_lt_handle(cuda, blas):
    """Applications pass a cublasHandle_t where a cublasLtHandle_t is expected (the reference's own test does,
    tests/cublas.cpp:447-452); both libraries share one context layout."""
    lt = capi.CublasLt()
    real = lt.handle
    lt.handle = blas.handle
    try:
        A, av = orc.fill_lcg("f32", 16 * 16, 1)
        Cz = np.zeros(256, dtype=np.float32)
        dA, dD = DeviceBuffer(cuda, A), DeviceBuffer(cuda, Cz)
        lt.matmul(N, N, 16, 16, 16, 1.0, dA.ptr, capi.CUDA_R_32F, 16, dA.ptr, capi.CUDA_R_32F, 16, 0.0, dD.ptr, capi.CUDA_R_32F, 16, dD.ptr,
                  capi.CUDA_R_32F, 16)
        a = av.reshape(16, 16).T.astype(np.float64)
        assert np.allclose(dD.download().reshape(16, 16).T, a @ a, atol=1e-4)
    finally:
        lt.handle = real
        lt.destroy()


# ---- Sgemv, Dgemm, batched pointers, aliased leading dimensions -------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("trans, m, n, incx, incy", [(N, 300, 77, 1, 1), (T, 130, 1000, 1, 1), (N, 65, 200, 3, 2), (T, 70, 129, 2, 5)])
def test_sgemv(cuda, blas, trans, m, n, incx, incy):
    lda = m + 3
    rows, cols = (n, m) if trans == T else (m, n)   # op(A) is rows x cols
    A, av = orc.fill_lcg("f32", lda * n, 1)
    x, xv = orc.fill_lcg("f32", cols * incx, 2)
    y, yv = orc.fill_lcg("f32", rows * incy, 3)
    dA, dx, dy = DeviceBuffer(cuda, A), DeviceBuffer(cuda, x), DeviceBuffer(cuda, y)
    blas.sgemv(trans, m, n, 0.5, dA.ptr, lda, dx.ptr, incx, -2.0, dy.ptr, incy)
    a = av.reshape(n, lda)[:, :m].T.astype(np.float64)      # m x n
    op = a.T if trans == T else a
    want = yv.astype(np.float64).copy()
    want[::incy][:rows] = 0.5 * (op @ xv[::incx][:cols].astype(np.float64)) - 2.0 * yv[::incy][:rows]
    got = dy.download()
    assert np.allclose(got, want, atol=1e-5 * math.sqrt(cols + 1) * max(1.0, np.abs(want).max()))  # strided gaps of y untouched too
    assert blas.last_path() == capi.PATH_GEMV
    assert blas.sgemv(N, 4, 4, 1.0, dA.ptr, 4, dx.ptr, -1, 0.0, dy.ptr, 1, check=False) == capi.STATUS_NOT_SUPPORTED   # negative increment
    assert blas.sgemv(N, 4, 4, 1.0, dA.ptr, 4, dx.ptr, 0, 0.0, dy.ptr, 1, check=False) == capi.STATUS_INVALID_VALUE
    assert blas.lib.cublasSgemv_v2_64(blas.handle, N, 1 << 32, 1, None, dA.ptr, 1 << 32, dx.ptr, 1, None, dy.ptr, 1) == capi.STATUS_NOT_SUPPORTED


@pytest.mark.gpu
@pytest.mark.parametrize("ta, tb", [(N, N), (T, N), (N, T), (T, T)])
def test_dgemm(cuda, blas, ta, tb):
    rng = np.random.default_rng(11)
    m, n, k = 67, 45, 130
    rows_a, cols_a = (k, m) if ta == T else (m, k)
    rows_b, cols_b = (n, k) if tb == T else (k, n)
    lda, ldb, ldc = rows_a + 3, rows_b + 1, m + 2
    A = rng.standard_normal(lda * cols_a)
    B = rng.standard_normal(ldb * cols_b)
    C0 = rng.standard_normal(ldc * n)
    dA, dB, dC = DeviceBuffer(cuda, A), DeviceBuffer(cuda, B), DeviceBuffer(cuda, C0)
    blas.dgemm(ta, tb, m, n, k, 1.25, dA.ptr, lda, dB.ptr, ldb, -0.5, dC.ptr, ldc)
    a = A.reshape(cols_a, lda)[:, :rows_a].T
    b = B.reshape(cols_b, ldb)[:, :rows_b].T
    want = C0.copy().reshape(n, ldc)
    want[:, :m] = (1.25 * ((a.T if ta == T else a) @ (b.T if tb == T else b)) - 0.5 * C0.reshape(n, ldc)[:, :m].T).T
    assert np.allclose(dC.download(), want.ravel(), rtol=0, atol=1e-12 * k)


@pytest.mark.gpu
def test_aliased_leading_dimension_sample(cuda, blas):
    """Leading dimensions that are multiples of 4 KiB (tests/cublas.cpp:550-585 checks every 7th row and column and the last)."""
    m, n, k, ld = 300, 264, 2048, 2048
    A, _ = orc.fill_lcg("f16", ld * m, 1)
    B, _ = orc.fill_lcg("f16", ld * n, 2)
    Cz = np.zeros(m * n, dtype=np.float32)
    dA, dB, dC = DeviceBuffer(cuda, A), DeviceBuffer(cuda, B), DeviceBuffer(cuda, Cz)
    blas.gemm_ex(T, N, m, n, k, 1.0, dA.ptr, capi.CUDA_R_16F, ld, dB.ptr, capi.CUDA_R_16F, ld, 0.0, dC.ptr, capi.CUDA_R_32F, m)
    rows = sorted(set(range(0, m, 7)) | {m - 1})
    cols = sorted(set(range(0, n, 7)) | {n - 1})
    want = orc.dots_fp64(True, False, k, A, "f16", ld, B, "f16", ld, rows, cols)
    got = dC.download().reshape(n, m).T[np.ix_(rows, cols)]
    assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max()) * math.sqrt(k + 1)
    assert blas.last_path() == capi.PATH_UMMA


@pytest.mark.gpu
def test_operand_shared_by_every_batch_entry(cuda, blas):
    """strideA = 0: one A for the whole batch (what cublasLtMatmul passes for a non-batched operand, cublasLt.cpp:381)."""
    m, n, k, batch = 128, 96, 64, 4
    A, av = orc.fill_lcg("f16", m * k, 1)
    B, bv = orc.fill_lcg("f16", k * n * batch, 2)
    Cz = np.zeros(m * n * batch, dtype=np.float32)
    dA, dB, dC = DeviceBuffer(cuda, A), DeviceBuffer(cuda, B), DeviceBuffer(cuda, Cz)
    blas.gemm_strided_batched_ex(T, N, m, n, k, 1.0, dA.ptr, capi.CUDA_R_16F, k, 0, dB.ptr, capi.CUDA_R_16F, k, k * n, 0.0, dC.ptr,
                                 capi.CUDA_R_32F, m, m * n, batch)
    a = av.reshape(m, k).astype(np.float64)
    want = np.stack([(a @ bv.reshape(batch, n, k)[e].astype(np.float64).T).T for e in range(batch)])
    assert np.allclose(dC.download().reshape(batch, n, m), want, atol=1e-4)


@pytest.mark.gpu
def test_split_along_k_gives_the_same_bits_every_time(cuda, blas):
    """A product that the tensor-core kernel splits along k (one tile pair, 128 k slices) sums its parts in split order, whichever
    part finishes last: twenty runs give one result, bit for bit, and it matches the fp64 reference."""
    import torch
    m, n, k = 256, 256, 8192
    A, av = orc.fill_lcg("f16", m * k, 31)
    B, bv = orc.fill_lcg("f16", n * k, 32)
    dA, dB = DeviceBuffer(cuda, A), DeviceBuffer(cuda, B)
    first = None
    for _ in range(20):
        dC = DeviceBuffer(cuda, np.zeros(m * n, dtype=np.float32))
        blas.gemm_ex(T, N, m, n, k, 1.0, dA.ptr, capi.CUDA_R_16F, k, dB.ptr, capi.CUDA_R_16F, k, 0.0, dC.ptr, capi.CUDA_R_32F, m)
        got = dC.download()
        assert blas.last_path() == capi.PATH_UMMA and blas.last_plan()["splits"] > 1, blas.last_plan()
        if first is None:
            first = got
            want = (av.reshape(m, k).astype(np.float64) @ bv.reshape(n, k).astype(np.float64).T).T.reshape(-1)
            assert np.max(np.abs(got - want) / np.maximum(1.0, np.abs(want))) <= 2e-3
        else:
            assert np.array_equal(got.view(np.uint32), first.view(np.uint32))
    assert blas.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1024, 4096, 520], ids=["rows of 2 KB", "rows of 8 KB", "rows of 1040 bytes"])
def test_matrix_vector_chain_between_copies_in_a_graph(cuda, n):
    """The matrix-vector kernel is launched so that it may start while the kernel before it drains. A chain y1 = M1 x,
    y2 = M2 y1, y3 = M3 y2 with a fill before it and a device-to-device copy in the middle, captured and replayed, must give
    what stream order gives: every link reads what the link before it wrote."""
    torch = cuda
    rng = np.random.default_rng(7)
    Ms = [torch.from_numpy((rng.standard_normal((n, n)) / math.sqrt(n)).astype(np.float16)).cuda() for _ in range(3)]
    x = torch.from_numpy(rng.standard_normal(n).astype(np.float16)).cuda()
    ys = [torch.zeros(n, dtype=torch.float16, device="cuda") for _ in range(4)]
    b = capi.Cublas()
    stream = torch.cuda.Stream()
    b.set_stream(stream.cuda_stream)

    def link(M, v, y):  # y = M v with M row-major n x n, i.e. op(A) = A^T of the column-major n x n matrix holding M^T
        b.gemm_ex(T, N, n, 1, n, 1.0, M.data_ptr(), capi.CUDA_R_16F, n, v.data_ptr(), capi.CUDA_R_16F, n, 0.0, y.data_ptr(), capi.CUDA_R_16F, n)
        assert b.last_path() == capi.PATH_GEMV

    def chain():
        ys[0].fill_(0)
        link(Ms[0], x, ys[0])
        link(Ms[1], ys[0], ys[1])
        ys[2].copy_(ys[1])
        link(Ms[2], ys[2], ys[3])

    with torch.cuda.stream(stream):
        chain()
        stream.synchronize()
        eager = ys[3].clone()
        for y in ys:
            y.zero_()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            chain()
        for _ in range(5):
            graph.replay()
        stream.synchronize()
    want = x.double()
    for M in Ms:
        want = (M.double() @ want).half().double()
    assert torch.equal(ys[3], eager)
    assert torch.allclose(ys[3].double(), want, rtol=2e-2, atol=2e-2)
    assert b.device_status() == 0
    b.destroy()


@pytest.mark.gpu
def test_gemm_grouped_batched_ex(cuda, blas):
    """cublasGemmGroupedBatchedEx as the reference's acceptance test calls it (tests/cublas.cpp:491-548): three groups of f16
    TN problems with fp32 C, each group with its own shape, scalars, leading dimensions and entry count; the pointer arrays
    list every problem group after group; scalars are arrays of float on the host (COMPUTE_32F_FAST_16F)."""
    groups = [(40, 7, 33, 2, 1.0, 0.0), (17, 5, 64, 1, -0.5, 1.0), (64, 1, 48, 3, 2.0, 0.0)]   # m, n, k, count, alpha, beta
    mats, seed = [], 11
    for (m, n, k, count, alpha, beta) in groups:
        for _ in range(count):
            A, av = orc.fill_lcg("f16", k * m, seed)
            B, bv = orc.fill_lcg("f16", k * n, seed + 1)
            Cm, cv = orc.fill_lcg("f32", m * n, seed + 2)
            seed += 3
            mats.append((DeviceBuffer(cuda, A), DeviceBuffer(cuda, B), DeviceBuffer(cuda, Cm), av, bv, cv))
    total = len(mats)
    ptrs = np.array([x[0].ptr for x in mats] + [x[1].ptr for x in mats] + [x[2].ptr for x in mats], dtype=np.uint64)
    dP = DeviceBuffer(cuda, ptrs)
    ints = lambda values: (C.c_int * len(values))(*values)
    floats = lambda values: (C.c_float * len(values))(*values)
    status = blas.lib.cublasGemmGroupedBatchedEx(
        blas.handle, ints([T] * 3), ints([N] * 3), ints([g[0] for g in groups]), ints([g[1] for g in groups]), ints([g[2] for g in groups]),
        floats([g[4] for g in groups]), dP.ptr, capi.CUDA_R_16F, ints([g[2] for g in groups]), dP.ptr + 8 * total, capi.CUDA_R_16F,
        ints([g[2] for g in groups]), floats([g[5] for g in groups]), dP.ptr + 16 * total, capi.CUDA_R_32F, ints([g[0] for g in groups]), 3,
        ints([g[3] for g in groups]), capi.COMPUTE_32F_FAST_16F)
    assert status == capi.STATUS_SUCCESS
    p = 0
    for (m, n, k, count, alpha, beta) in groups:
        for _ in range(count):
            dA, dB, dC, av, bv, cv = mats[p]
            a = av.reshape(m, k).astype(np.float64)            # A stored k x m: op(A) = A^T is m x k
            b = bv.reshape(n, k).astype(np.float64)
            want = alpha * (a @ b.T) + beta * cv.reshape(n, m).T.astype(np.float64)
            got = dC.download().reshape(n, m).T
            assert (np.abs(got - want) <= 2e-3 * np.maximum(1.0, np.abs(want)) * 8.0).all(), f"problem {p}"   # tests/cublas.cpp:537
            p += 1
    # argument checks of the entry point itself
    assert blas.lib.cublasGemmGroupedBatchedEx(blas.handle, None, None, None, None, None, None, 0, capi.CUDA_R_16F, None, 0, capi.CUDA_R_16F,
                                               None, None, 0, capi.CUDA_R_32F, None, 0, None, capi.COMPUTE_32F) == capi.STATUS_SUCCESS
    assert blas.lib.cublasGemmGroupedBatchedEx(blas.handle, None, None, None, None, None, None, 0, capi.CUDA_R_16F, None, 0, capi.CUDA_R_16F,
                                               None, None, 0, capi.CUDA_R_32F, None, 2, None, capi.COMPUTE_32F) == capi.STATUS_INVALID_VALUE


@pytest.mark.gpu
def test_more_columns_than_one_grid_dimension_holds(cuda, blas):
    """k = 0 scales C by beta for a result with 300000 columns (a grid dimension holds 65535 blocks), and a thin fp32 product
    of the same width goes through the tile kernels' column chunks."""
    m, n = 4, 300000
    C0, cv = orc.fill_lcg("f32", m * n, 5)
    dC = DeviceBuffer(cuda, C0)
    blas.sgemm(N, N, m, n, 0, 1.0, dC.ptr, m, dC.ptr, 1, 0.5, dC.ptr, m)
    assert blas.last_path() == capi.PATH_SCALE
    assert np.array_equal(dC.download(), (0.5 * cv).astype(np.float32))
    k = 3
    A, av = orc.fill_lcg("f32", m * k, 6)
    B, bv = orc.fill_lcg("f32", k * n, 7)
    dA, dB, dD = DeviceBuffer(cuda, A), DeviceBuffer(cuda, B), DeviceBuffer(cuda, np.zeros(m * n, dtype=np.float32))
    blas.sgemm(N, N, m, n, k, 1.0, dA.ptr, m, dB.ptr, k, 0.0, dD.ptr, m)
    want = (av.reshape(k, m).T.astype(np.float64) @ bv.reshape(n, k).T.astype(np.float64)).T.ravel()
    assert np.allclose(dD.download(), want, atol=1e-5)


# ---- pointer-array batches on the tensor cores ---------------------------------------------------------------------------

POINTER_CASES = [
    # name, ta, tb, m, n, k, type ab, type c, alpha, beta, batch, byte offset of entry 1's A (0: aligned)
    ("f16 TN -> f32", T, N, 256, 192, 128, "f16", "f32", 1.0, 0.0, 24, 0),
    ("bf16 NN -> bf16 with beta", N, N, 128, 136, 256, "bf16", "bf16", 0.5, 1.5, 16, 0),
    ("f16 NT ragged -> f16", N, T, 200, 72, 192, "f16", "f16", 1.0, 0.0, 20, 0),
    ("int8 TN -> s32", T, N, 256, 128, 512, "s8", "s32", 1, 0, 12, 0),
    ("f16 TN, one entry not 16-byte aligned", T, N, 256, 192, 128, "f16", "f32", 1.0, 0.5, 24, 2),
    ("f16 TN, C rows not a multiple of 16 bytes (direct stores)", T, N, 250, 64, 128, "f16", "f32", 1.0, 0.0, 24, 0),
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", POINTER_CASES, ids=lambda c: c[0])
def test_pointer_array_batch_on_tensor_cores(cuda, blas, case):
    """cublasGemmBatchedEx with aligned matrices runs on the tcgen05 kernel through per-entry tensor maps built on the device
    (the reference serves pointer arrays from its scalar shader, src/cublas/cublas.cpp:787, 1131-1139). Whether an entry's
    address suits TMA only the device can tell: when one does not, the CUDA-core kernel queued behind does the work instead,
    and the results are the same either way."""
    from vulkanizer_b200 import synth
    name, ta, tb, m, n, k, kind, kind_c, alpha, beta, batch, misalign = case
    rows_a, cols_a = (k, m) if ta == T else (m, k)
    rows_b, cols_b = (n, k) if tb == T else (k, n)
    lda, ldb, ldc = (rows_a + 7) // 8 * 8, (rows_b + 7) // 8 * 8, m
    es, es_c = ELEM[kind], ELEM[kind_c]
    pitch_a, pitch_b, pitch_c = lda * cols_a + 64, ldb * cols_b + 64, ldc * n + 64   # entries lie apart, each 16-byte aligned
    if kind == "s8":
        A, B = synth.int8_uniform(2, pitch_a * batch), synth.int8_uniform(2, pitch_b * batch, first=1 << 20)
        C0 = (synth.int8_uniform(9, pitch_c * batch).astype(np.int32)) * 100
    else:
        A, _ = orc.fill_lcg(kind, pitch_a * batch, 51)
        B, _ = orc.fill_lcg(kind, pitch_b * batch, 52)
        C0, _ = orc.fill_lcg(kind_c, pitch_c * batch, 53)
    dA, dB, dC = DeviceBuffer(cuda, A), DeviceBuffer(cuda, B), DeviceBuffer(cuda, C0)
    offs_a = [e * pitch_a * es + (misalign if e == 1 else 0) for e in range(batch)]
    ptrs = np.array([dA.ptr + o for o in offs_a] + [dB.ptr + e * pitch_b * es for e in range(batch)] + [dC.ptr + e * pitch_c * es_c for e in range(batch)],
                    dtype=np.uint64)
    dP = DeviceBuffer(cuda, ptrs)
    compute = capi.COMPUTE_32I if kind == "s8" else capi.COMPUTE_32F
    blas.gemm_batched_ex(ta, tb, m, n, k, alpha, dP.ptr, CUDA_TYPE[kind], lda, dP.ptr + 8 * batch, CUDA_TYPE[kind], ldb, beta, dP.ptr + 16 * batch,
                         CUDA_TYPE[kind_c], ldc, batch, compute=compute)
    assert blas.last_path() == capi.PATH_UMMA
    got_all = dC.download()
    for e in (0, 1, batch - 1):
        a0 = offs_a[e] // es
        Ae, Be, Ce = A[a0:a0 + lda * cols_a], B[e * pitch_b:e * pitch_b + ldb * cols_b], C0[e * pitch_c:e * pitch_c + ldc * n]
        got = got_all[e * pitch_c:e * pitch_c + ldc * n]
        if kind == "s8":
            want = orc.gemm_s8(ta == T, tb == T, m, n, k, 1, alpha, np.ascontiguousarray(Ae), lda, 0, np.ascontiguousarray(Be), ldb, 0, beta, Ce.copy(), ldc, 0)
            assert np.array_equal(got, want), f"entry {e}"
        else:
            want, _ = orc.gemm_fp64(ta == T, tb == T, m, n, k, 1, alpha, np.ascontiguousarray(Ae), kind, lda, 0, np.ascontiguousarray(Be), kind, ldb, 0, beta,
                                    np.ascontiguousarray(Ce), kind_c, ldc, 0)
            rel = 1e-5 if kind_c == "f32" else 2e-3 if kind_c == "f16" else 1.6e-2
            tol = rel * np.maximum(1.0, np.abs(want)) * math.sqrt(k + 1.0)
            assert (np.abs(orc.to_float(got, kind_c) - want) <= tol).all(), f"entry {e}"
    # the gaps between the entries of C are untouched
    for e in range(batch):
        assert np.array_equal(got_all[e * pitch_c + ldc * n:(e + 1) * pitch_c], C0[e * pitch_c + ldc * n:(e + 1) * pitch_c])
    assert blas.device_status() == 0
