"""The five benchmark configurations at their full sizes, through the C ABI, checked on samples and by properties.

Full fp64 references for 8192^3 would take the CPU minutes to hours, so, like k0zi/Vulkanizer's own large test
(tests/cublas.cpp:550-585: every 7th row and column plus the last), results are compared with fp64 dot products on a sample of
rows and columns, and the whole result is tied down with size-independent properties: a checksum identity
(sum over rows of D equals (sum over rows of op(A)) * op(B)) and linearity in alpha. Tolerances are those stated for the
configurations: 1e-5 relative for fp32 FFMA, 1e-2 for f16 / bf16 (against fp64), exact for int8.
"""
import math

import numpy as np
import pytest

from harness import DeviceBuffer, N, T
from oracle import pyoracle as orc
from vulkanizer_b200 import capi, synth


def to_f16(v):
    return v.astype(np.float16).view(np.uint16)


def sample_indices(size, step=509):
    return sorted(set(range(0, size, step)) | {size - 1})


@pytest.fixture(scope="module")
def blas(cuda):
    b = capi.Cublas()
    yield b
    b.destroy()


@pytest.mark.gpu
def test_config1_sgemm_512_full_reference(cuda, blas):
    """cublasSgemm NN 512^3, alpha = 1, beta = 0.5, uniform[-1, 1], seed 0: whole result against fp64 and the reference's CPU GEMM."""
    n = 512
    A, B, C0 = synth.uniform(0, n * n), synth.uniform(0, n * n, first=n * n), synth.uniform(0, n * n, first=2 * n * n)
    want, _ = orc.gemm_fp64(False, False, n, n, n, 1, 1.0, A, "f32", n, 0, B, "f32", n, 0, 0.5, C0, "f32", n, 0)
    cpu = orc.gemm_f32(False, False, n, n, n, 1, 1.0, A, "f32", n, 0, B, "f32", n, 0, 0.5, C0.copy(), "f32", n, 0)
    dA, dB, dC = DeviceBuffer(cuda, A), DeviceBuffer(cuda, B), DeviceBuffer(cuda, C0)
    blas.sgemm(N, N, n, n, n, 1.0, dA.ptr, n, dB.ptr, n, 0.5, dC.ptr, n)
    got = dC.download()
    assert blas.last_path() == capi.PATH_SGEMM
    rel = np.abs(got - want) / np.maximum(1.0, np.abs(want))
    assert rel.max() <= 1e-5, rel.max()
    # the reference's own CPU result differs from fp64 by its fp32 summation order; ours must be as close to it as to fp64
    assert (np.abs(got - cpu) / np.maximum(1.0, np.abs(cpu))).max() <= 2e-5


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_config2_gemmex_8192(cuda, blas, kind):
    """cublasGemmEx TN 8192^3, f16 / bf16 -> f32, normal(0, 0.02), seed 1."""
    torch = cuda
    n = 8192
    a = synth.normal(1, n * n, 0.02)
    b = synth.normal(1, n * n, 0.02, first=n * n)
    A, B = orc.to_storage(a, kind), orc.to_storage(b, kind)
    del a, b
    tdt = torch.float16 if kind == "f16" else torch.bfloat16
    dA = torch.from_numpy(A.view(np.int16)).cuda().view(tdt)
    dB = torch.from_numpy(B.view(np.int16)).cuda().view(tdt)
    dC = torch.full((n * n,), float("nan"), dtype=torch.float32, device="cuda")
    t = capi.CUDA_R_16F if kind == "f16" else capi.CUDA_R_16BF
    blas.gemm_ex(T, N, n, n, n, 1.0, dA.data_ptr(), t, n, dB.data_ptr(), t, n, 0.0, dC.data_ptr(), capi.CUDA_R_32F, n)
    torch.cuda.synchronize()
    assert blas.last_path() == capi.PATH_UMMA and blas.device_status() == 0
    rows, cols = sample_indices(n), sample_indices(n, 1021)
    want = orc.dots_fp64(True, False, n, A, kind, n, B, kind, n, rows, cols)
    D = dC.view(n, n)  # [col, row]
    got = D[torch.tensor(cols, device="cuda")][:, torch.tensor(rows, device="cuda")].T.cpu().numpy().astype(np.float64)
    scale = np.maximum(1.0, np.abs(want))
    assert (np.abs(got - want) / scale).max() <= 1e-2
    # every entry was written, and the checksum identity holds over the whole matrix: 1^T D = (A 1)^T B
    assert torch.isfinite(dC).all()
    colsum = D.double().sum(dim=1)                                   # sum over rows, per column
    asum = dA.view(n, n).double().sum(dim=0)                         # sum over i of A(l, i): a k-vector
    ref = dB.view(n, n).double() @ asum                              # per column j: sum_l B(l, j) asum(l)
    assert torch.allclose(colsum, ref, rtol=0, atol=1e-3 * float(ref.abs().max()) + 1e-2)
    # linearity in alpha and beta on a second call: D2 = 2 * product + 0.5 * D
    blas.gemm_ex(T, N, n, n, n, 2.0, dA.data_ptr(), t, n, dB.data_ptr(), t, n, 0.5, dC.data_ptr(), capi.CUDA_R_32F, n)
    torch.cuda.synchronize()
    got2 = D[torch.tensor(cols, device="cuda")][:, torch.tensor(rows, device="cuda")].T.cpu().numpy().astype(np.float64)
    assert (np.abs(got2 - 2.5 * want) / np.maximum(1.0, np.abs(2.5 * want))).max() <= 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("m, n, k", [(11008, 512, 4096), (4096, 512, 11008)])
def test_config3_int8_projection_shapes_bit_exact(cuda, blas, m, n, k):
    """cublasGemmEx TN int8 -> int32, uniform integers in [-127, 127], seed 2: the whole result, bit for bit."""
    torch = cuda
    A = synth.int8_uniform(2, m * k)
    B = synth.int8_uniform(2, k * n, first=m * k)
    want = orc.gemm_s8(True, False, m, n, k, 1, 1, A, k, 0, B, k, 0, 0, np.zeros(m * n, dtype=np.int32), m, 0)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.full((m * n,), -7, dtype=torch.int32, device="cuda")
    blas.gemm_ex(T, N, m, n, k, 1, dA.data_ptr(), capi.CUDA_R_8I, k, dB.data_ptr(), capi.CUDA_R_8I, k, 0, dC.data_ptr(), capi.CUDA_R_32I, m,
                 capi.COMPUTE_32I)
    torch.cuda.synchronize()
    assert blas.last_path() == capi.PATH_UMMA and blas.device_status() == 0
    assert np.array_equal(dC.cpu().numpy(), want)
    assert np.abs(want).max() < 2 ** 31 - 1


@pytest.mark.gpu
def test_config4_batched_attention_scores(cuda, blas):
    """cublasGemmStridedBatchedEx TN, batch 256, M = N = 1024, K = 128, alpha = 1/sqrt(128), f16 -> f32, normal(0, 1), seed 3."""
    torch = cuda
    batch, m, n, k = 256, 1024, 1024, 128
    alpha = 1.0 / math.sqrt(128.0)
    A = to_f16(synth.normal(3, batch * m * k))
    B = to_f16(synth.normal(3, batch * n * k, first=batch * m * k))
    dA = torch.from_numpy(A.view(np.int16)).cuda().view(torch.float16)
    dB = torch.from_numpy(B.view(np.int16)).cuda().view(torch.float16)
    dC = torch.full((batch * m * n,), float("nan"), dtype=torch.float32, device="cuda")
    blas.gemm_strided_batched_ex(T, N, m, n, k, alpha, dA.data_ptr(), capi.CUDA_R_16F, k, m * k, dB.data_ptr(), capi.CUDA_R_16F, k, n * k, 0.0,
                                 dC.data_ptr(), capi.CUDA_R_32F, m, m * n, batch)
    torch.cuda.synchronize()
    assert blas.last_path() == capi.PATH_UMMA and blas.device_status() == 0
    assert torch.isfinite(dC).all()
    # three whole batch entries against the fp64 reference (first, one in the middle, last)
    for e in (0, 131, 255):
        want, _ = orc.gemm_fp64(True, False, m, n, k, 1, alpha, A[e * m * k:(e + 1) * m * k], "f16", k, 0, B[e * n * k:(e + 1) * n * k], "f16", k, 0,
                                0.0, np.zeros(m * n, dtype=np.float32), "f32", m, 0)
        got = dC[e * m * n:(e + 1) * m * n].cpu().numpy()
        assert (np.abs(got - want) / np.maximum(1.0, np.abs(want))).max() <= 1e-2
    # the checksum identity over every entry: 1^T D_e = alpha (A_e 1)^T B_e
    D = dC.view(batch, n, m).double()
    asum = dA.view(batch, m, k).double().sum(dim=1)                             # (batch, k)
    ref = alpha * torch.einsum("bnk,bk->bn", dB.view(batch, n, k).double(), asum)
    assert torch.allclose(D.sum(dim=2), ref, rtol=0, atol=1e-3 * float(ref.abs().max()) + 1e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("m", [4096, 11008])
def test_config5a_decode_gemv(cuda, blas, m):
    """cublasGemmEx TN with N = 1, K = 4096: fp16 weights normal(0, 0.02), fp32 result, seed 4: whole result."""
    torch = cuda
    k = 4096
    W = to_f16(synth.normal(4, m * k, 0.02))
    x = to_f16(synth.normal(4, k, 1.0, first=m * k))
    want, _ = orc.gemm_fp64(True, False, m, 1, k, 1, 1.0, W, "f16", k, 0, x, "f16", k, 0, 0.0, np.zeros(m, dtype=np.float32), "f32", m, 0)
    dW, dx, dy = DeviceBuffer(cuda, W), DeviceBuffer(cuda, x), DeviceBuffer(cuda, np.zeros(m, dtype=np.float32))
    blas.gemm_ex(T, N, m, 1, k, 1.0, dW.ptr, capi.CUDA_R_16F, k, dx.ptr, capi.CUDA_R_16F, k, 0.0, dy.ptr, capi.CUDA_R_32F, m)
    got = dy.download()
    assert blas.last_path() == capi.PATH_GEMV
    assert (np.abs(got - want) / np.maximum(1.0, np.abs(want))).max() <= 1e-2
    assert np.abs(got - want).max() <= 1e-4 * math.sqrt(k)  # fp32 accumulation of exact fp16 products: far inside the 1e-2 bar


@pytest.mark.gpu
def test_config5b_lt_matmul_bf16_column_block(cuda):
    """cublasLtMatmul bf16 -> f32 on one rank's share of the N-sharded product, at a size the check can afford:
    M = K = 4096 and a 1024-column block written in place into a wider D (ldd = M), as the sharded run does."""
    torch = cuda
    m, k, width, n_total = 4096, 4096, 1024, 4096
    A = orc.to_storage(synth.normal(5, m * k), "bf16")
    B = orc.to_storage(synth.normal(5, width * k, first=m * k), "bf16")
    dA = torch.from_numpy(A.view(np.int16)).cuda().view(torch.bfloat16)
    dB = torch.from_numpy(B.view(np.int16)).cuda().view(torch.bfloat16)
    D = torch.full((n_total * m,), 7.0, dtype=torch.float32, device="cuda")
    first = 2048  # this block's first column
    lt = capi.CublasLt()
    ptr = D.data_ptr() + 4 * first * m
    lt.matmul(T, N, m, width, k, 1.0, dA.data_ptr(), capi.CUDA_R_16BF, k, dB.data_ptr(), capi.CUDA_R_16BF, k, 0.0, ptr, capi.CUDA_R_32F, m, ptr,
              capi.CUDA_R_32F, m)
    torch.cuda.synchronize()
    assert lt.last_path() == capi.PATH_UMMA
    rows, cols = sample_indices(m, 257), sample_indices(width, 101)
    want = orc.dots_fp64(True, False, k, A, "bf16", k, B, "bf16", k, rows, cols)
    Dm = D.view(n_total, m)
    got = Dm[first:first + width][torch.tensor(cols, device="cuda")][:, torch.tensor(rows, device="cuda")].T.cpu().numpy()
    assert (np.abs(got - want) / np.maximum(1.0, np.abs(want))).max() <= 1e-2
    assert bool((Dm[:first] == 7.0).all()) and bool((Dm[first + width:] == 7.0).all()), "columns outside the block must stay untouched"
    lt.destroy()


@pytest.mark.gpu
def test_config5b_full_height_column_block(cuda):
    """The sharded product at its real height and depth: M = K = 32768 (A is 2 GiB of bf16) and one 256-column block of the
    32768-column result, operands from the seeded generator's torch form, checked against the fp64 oracle on rows spread over
    the whole height with the operands regenerated on the host by the numpy form (seed 5: value i of the stream for element i of
    A^T's storage, value m k + i for element i of B)."""
    torch = cuda
    free, _ = torch.cuda.mem_get_info()
    if free < (8 << 30):
        pytest.skip("needs 8 GiB of free device memory")
    m = k = 32768
    width, first_col = 256, 20480   # a block from the middle of the result
    A = torch.empty(m * k, dtype=torch.bfloat16, device="cuda")
    synth.fill_normal_torch(torch, A, 5, 1.0, first=0)
    B = torch.empty(width * k, dtype=torch.bfloat16, device="cuda")
    synth.fill_normal_torch(torch, B, 5, 1.0, first=m * k + first_col * k)
    D = torch.zeros(width * m, dtype=torch.float32, device="cuda")
    lt = capi.CublasLt()
    lt.matmul(T, N, m, width, k, 1.0, A.data_ptr(), capi.CUDA_R_16BF, k, B.data_ptr(), capi.CUDA_R_16BF, k, 0.0, D.data_ptr(), capi.CUDA_R_32F, m, D.data_ptr(),
              capi.CUDA_R_32F, m)
    torch.cuda.synchronize()
    assert lt.last_path() == capi.PATH_UMMA
    rows, cols = sample_indices(m, 1021), [0, 100, 255]
    a_rows = np.concatenate([orc.to_storage(synth.normal(5, k, 1.0, first=i * k), "bf16") for i in rows])
    b_cols = np.concatenate([orc.to_storage(synth.normal(5, k, 1.0, first=m * k + (first_col + j) * k), "bf16") for j in cols])
    # what the device holds for those rows and columns is what the host form of the generator gives
    assert np.array_equal(A.view(torch.int16).view(m, k)[torch.tensor(rows, device="cuda")].cpu().numpy().view(np.uint16).ravel(), a_rows)
    want = orc.dots_fp64(True, False, k, a_rows, "bf16", k, b_cols, "bf16", k, list(range(len(rows))), list(range(len(cols))))
    got = D.view(width, m)[torch.tensor(cols, device="cuda")][:, torch.tensor(rows, device="cuda")].T.cpu().numpy()
    assert (np.abs(got - want) / np.maximum(1.0, np.abs(want))).max() <= 1e-2
    # and the whole block through the checksum identity: 1^T D = (A 1)^T B, columns of D summed over all 32768 rows
    asum = torch.zeros(k, dtype=torch.float64, device="cuda")      # sum over rows of op(A): length k, 2048 rows at a time
    for i in range(0, m, 2048):
        asum += A.view(m, k)[i:i + 2048].double().sum(dim=0)
    ref = B.view(width, k).double() @ asum
    assert torch.allclose(D.view(width, m).double().sum(dim=1), ref, rtol=0, atol=1e-3 * float(ref.abs().max()) + 1.0)
    lt.destroy()
