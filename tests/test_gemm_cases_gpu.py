"""Parity of the CUDA paths with the oracle on the case table of the reference's acceptance test.

Every row of k0zi/Vulkanizer's tests/cublas.cpp:598-682 is run through this repository's libcublas.so.12 with the
same LCG data, padded leading dimensions and tolerance (harness.py), and compared with the fp64 reference of that
test. Cases that only fp32 accumulation order separates from the reference's own CPU GEMM are also compared with
it (oracle_gemm_f32, pinned bit for bit against the compiled reference) at a tolerance of 1e-5 * sqrt(k) relative.
"""
import numpy as np
import pytest

from harness import Case, N, T, run_case
from vulkanizer_b200 import capi

F32, F16, BF16 = "f32", "f16", "bf16"
C16, FAST16 = capi.COMPUTE_16F, capi.COMPUTE_32F_FAST_16F
C32 = capi.COMPUTE_32F

CASES = [
    Case("sgemm NN", N, N, 70, 33, 129, F32, F32, F32, 1.0, 0.0),
    Case("sgemm TN", T, N, 128, 64, 64, F32, F32, F32, 0.5, 0.0),
    Case("sgemm NT beta", N, T, 65, 65, 17, F32, F32, F32, -1.0, 2.0),
    Case("sgemm TT", T, T, 3, 200, 300, F32, F32, F32, 1.0, 1.0),
    Case("gemmEx f16 -> f32", T, N, 96, 40, 256, F16, F16, F32, 1.0, 0.0),
    Case("gemmEx f16 -> f16", T, N, 64, 64, 64, F16, F16, F16, 1.0, 0.0),
    Case("gemmEx f16 tn fast", T, N, 200, 137, 72, F16, F16, F16, 0.5, -1.0, 1, C32, True),
    Case("gemmEx f16 tn fast f32 C", T, N, 130, 129, 37, F16, F16, F32, 1.0, 0.25, 1, C32, True),
    Case("gemmEx f16 tn 16F", T, N, 257, 130, 300, F16, F16, F16, 1.0, 0.5, 1, C16, True),
    Case("gemmEx f16 tn 16F f32 C", T, N, 64, 200, 45, F16, F16, F32, -2.0, 0.0, 1, FAST16, True),
    Case("strided f16 tn 16F", T, N, 128, 64, 128, F16, F16, F16, 1.0, 0.0, 7, C16, True),
    Case("gemmEx f16 tn large", T, N, 1030, 777, 72, F16, F16, F16, 0.5, -1.0, 1, C32, True),
    Case("gemmEx f16 tn large f32 C", T, N, 1100, 520, 40, F16, F16, F32, 1.0, 0.25, 1, C32, True),
    Case("coop f16 NN large", N, N, 1030, 777, 72, F16, F16, F16, 0.5, -1.0, 1, C32, True),
    Case("coop f16 NT large f32 C", N, T, 1100, 520, 40, F16, F16, F32, 1.0, 0.25, 1, C32, True),
    Case("coop f16 TT strided", T, T, 300, 260, 136, F16, F16, F16, 1.0, 0.0, 3, C32, True),
    Case("coop f16 NN strided k % 8", N, N, 128, 300, 77, F16, F16, F16, 1.0, 0.0, 4, C32, True),
    Case("coop bf16 TN -> f32 large", T, N, 520, 390, 100, BF16, BF16, F32, 1.0, 0.5, 1, C32, True),
    Case("coop bf16 NN -> bf16", N, N, 300, 260, 64, BF16, BF16, BF16, 1.0, -0.5, 2, C32, True),
    Case("coop bf16 NT -> bf16 large", N, T, 1030, 640, 48, BF16, BF16, BF16, 0.5, 0.0, 1, C32, True),
    Case("coop f16 TN long k f32 C", T, N, 264, 136, 4104, F16, F16, F32, 1.0, 0.5, 1, C32, True),
    Case("coop f16 NN long k", N, N, 264, 200, 4104, F16, F16, F16, 1.0, 0.0, 1, C32, True),
    Case("split along k f16 TN f32 C beta", T, N, 256, 300, 4096, F16, F16, F32, 1.0, 0.5, 1, C32, True),
    Case("split along k bf16 NN -> bf16", N, N, 512, 256, 2048, BF16, BF16, BF16, 0.5, 0.0, 1, C32, True),
    Case("split along k f16 TN odd rows (direct stores)", T, N, 250, 130, 3072, F16, F16, F16, 1.0, 0.0, 1, C32, True),
    Case("gemmEx f16 tn odd ld", T, N, 130, 129, 37, F16, F16, F32, 1.0, 0.25),
    Case("gemmEx bf16 -> f32", N, N, 50, 70, 90, BF16, BF16, F32, 1.0, 0.0),
    Case("gemmEx f16 x f32", T, N, 33, 31, 100, F16, F32, F32, 1.0, 0.0),
    Case("strided batched f16", T, N, 64, 16, 128, F16, F16, F16, 1.0, 0.0, 12),
    Case("pointer batched f32", T, N, 40, 24, 64, F32, F32, F32, 1.0, 0.0, -5),
    Case("gemv NN f32", N, N, 300, 1, 77, F32, F32, F32, 1.0, 0.0),
    Case("gemv TN f32 beta", T, N, 130, 1, 1000, F32, F32, F32, 0.5, -2.0),
    Case("gemv NT f16", N, T, 65, 1, 200, F16, F16, F16, 1.0, 0.0),
    Case("gemv TT bf16 -> f32", T, T, 70, 1, 129, BF16, BF16, F32, 1.0, 1.0),
    Case("gemv m=1 NN", N, N, 1, 333, 90, F32, F32, F32, 1.0, 0.5),
    Case("gemv m=1 TT f16", T, T, 1, 70, 257, F16, F16, F32, -1.0, 0.0),
    Case("gemv m=1 NT", N, T, 1, 40, 64, F32, F32, F32, 1.0, 0.0),
    Case("gemv m=1 TN f16 x f32", T, N, 1, 50, 31, F16, F32, F32, 2.0, 0.0),
    Case("gemv 1x1", T, N, 1, 1, 500, F32, F32, F32, 1.0, 0.0),
    Case("gemv strided batched f16", T, N, 129, 1, 128, F16, F16, F16, 1.0, 0.0, 9, C16),
    Case("gemv f16 aligned rows", T, N, 100, 1, 203, F16, F16, F32, 1.0, 0.5, 3, C32, True),
    Case("gemv f16 long rows", T, N, 33, 1, 3000, F16, F32, F16, 1.0, 0.0, 1, C32, True),
    Case("gemv bulk f16 one piece", T, N, 300, 1, 4096, F16, F16, F16, 1.0, 0.5, 1, C32, True),
    Case("gemv bulk bf16 three pieces", T, N, 1000, 1, 11008, BF16, BF16, F32, 0.5, 0.0, 1, C32, True),
    Case("gemv bulk f16 one chunk", T, N, 77, 1, 8, F16, F16, F32, 1.0, 0.0, 1, C32, True),
    Case("gemv bulk f16 ragged piece", T, N, 150, 1, 4104, F16, F16, F16, -1.0, 0.0, 1, C32, True),
    Case("gemv bulk bf16 fewer rows than SMs", T, N, 3, 1, 24064, BF16, BF16, BF16, 1.0, 1.0, 1, C32, True),
    Case("gemv bulk f16 many short rows", T, N, 5000, 1, 520, F16, F16, F16, 1.0, 0.0, 1, C32, True),
    Case("gemv bulk m=1 NN f16", N, N, 1, 500, 1024, F16, F16, F16, 1.0, 0.0, 1, C32, True),
    Case("two columns on the matrix-vector kernel, f16", T, N, 300, 2, 4096, F16, F16, F16, 1.0, 0.0, 1, C32, True),
    Case("two columns on the matrix-vector kernel, bf16 -> f32, beta", T, N, 1000, 2, 11008, BF16, BF16, F32, 0.5, -1.0, 1, C32, True),
    Case("two columns on the matrix-vector kernel, ragged piece", T, N, 150, 2, 4104, F16, F16, F16, -1.0, 0.0, 1, C32, True),
    Case("two columns on the matrix-vector kernel, short rows", T, N, 5000, 2, 520, F16, F16, F32, 1.0, 0.0, 1, C32, True),
    Case("three columns stay on the tensor cores", T, N, 300, 3, 4096, F16, F16, F16, 1.0, 0.0, 1, C32, True),
    Case("gemv pointer batched", T, N, 100, 1, 64, F32, F32, F32, 1.0, 0.0, -6),
    Case("gemv m=1 pointer batched", N, N, 1, 100, 64, F32, F32, F32, 1.0, 0.0, -4),
    Case("k = 0 scales C", N, N, 10, 10, 0, F32, F32, F32, 1.0, 3.0),
    Case("tiled NN", N, N, 200, 300, 77, F32, F32, F32, 1.0, -0.5),
    Case("tiled TN vec", T, N, 256, 384, 64, F32, F32, F32, 1.0, 0.0, 1, C32, True),
    Case("tiled NT vec", N, T, 136, 264, 40, F32, F32, F32, 0.5, 1.0, 1, C32, True),
    Case("tiled TT", T, T, 129, 131, 300, F32, F32, F32, 1.0, 0.0),
    Case("tiled NN vec A, k % 8", N, N, 200, 130, 100, F32, F32, F32, 1.0, 2.0, 1, C32, True),
    Case("tiled f16 NN vec", N, N, 192, 200, 96, F16, F16, F16, 1.0, 0.5, 1, C32, True),
    Case("tiled bf16 NT -> f32", N, T, 140, 150, 33, BF16, BF16, F32, 1.0, 0.0),
    Case("tiled f16 x f32 TT vec", T, T, 256, 128, 80, F16, F32, F32, -1.0, 0.0, 1, C32, True),
    Case("tiled bf16 TN -> bf16", T, N, 160, 144, 48, BF16, BF16, BF16, 1.0, 0.0, 1, C32, True),
    Case("tiled strided NN vec", N, N, 128, 136, 64, F32, F32, F32, 1.0, 0.0, 3, C32, True),
    Case("tiled pointers f16 NT", N, T, 130, 140, 50, F16, F16, F32, 1.0, 0.0, -3),
]


@pytest.fixture(scope="module")
def blas(cuda):
    b = capi.Cublas()
    yield b
    b.destroy()


def check(c, got, want, tol, before):
    bad = ~(np.abs(got - want) <= tol)
    assert not bad.any(), f"{c.name}: {int(bad.sum())} of {got.size} wrong, first at {int(np.argmax(bad))}: " \
                          f"got {got[np.argmax(bad)]}, want {want[np.argmax(bad)]}"


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=str)
def test_reference_case_table(cuda, blas, case):
    got, want, tol, before, path = run_case(cuda, blas, case)
    check(case, got, want, tol, before)
    assert blas.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("case", [c for c in CASES if c.aligned and c.type_a == c.type_b and c.type_a != F32 and c.m > 1 and c.n > 2],
                         ids=str)
def test_aligned_16bit_cases_run_on_tensor_cores(cuda, blas, case):
    """What the reference sends to its cooperative-matrix or f16 kernels (16-byte aligned f16 / bf16 operands) must take
    the tcgen05 kernel here, in every transpose combination, not the CUDA-core fallback."""
    *_, path = run_case(cuda, blas, case)
    assert path == capi.PATH_UMMA


@pytest.mark.gpu
@pytest.mark.parametrize("case", [c for c in CASES if c.name.startswith("two columns on the matrix-vector kernel")], ids=str)
def test_two_column_products_stream_the_matrix_once(cuda, blas, case):
    """n = 2 with a k-contiguous 16-bit A is bound by reading A: it takes the matrix-vector kernel with two right-hand sides."""
    got, want, tol, before, path = run_case(cuda, blas, case)
    check(case, got, want, tol, before)
    assert path == capi.PATH_GEMV


@pytest.mark.gpu
@pytest.mark.parametrize("case", [c for c in CASES if c.type_a == c.type_b == c.type_c == F32 and c.batch >= 1], ids=str)
def test_fp32_cases_tf32_mode(cuda, case):
    """The reference's test sets CUBLAS_TF32_TENSOR_OP_MATH on its handle (tests/cublas.cpp:595); its data are exact in
    TF32, so the same tolerance must hold on the TF32 tensor-core path."""
    b = capi.Cublas()
    b.set_math_mode(capi.TF32_TENSOR_OP_MATH)
    try:
        got, want, tol, before, path = run_case(cuda, b, case)
        check(case, got, want, tol, before)
        assert b.device_status() == 0
    finally:
        b.destroy()
