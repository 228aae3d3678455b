"""cublasLtMatmul beyond the reference's six epilogues: auxiliary outputs (RELU_AUX, GELU_AUX), the backward epilogues (DRELU,
DGELU, with BGRAD), the operand bias gradients (BGRADA, BGRADB) and matrices in row order.

k0zi/Vulkanizer answers NOT_SUPPORTED for all of these (src/cublas/cublasLt.cpp:68-78, 83), so there is no reference result to
match: the expected values are NVIDIA's documented semantics (include/vkzb_cublaslt.h states them) computed in fp64 with
numpy, held to the tolerance of the reference's cuBLASLt test (tests/cublas.cpp:470: 1e-5, or 4e-3 for half, times sqrt(k)).
Every shape runs once on a small unaligned problem (CUDA-core kernels, per-element epilogue) and once on an aligned one that
takes the tcgen05 kernel's staged epilogue.
"""
import math

import numpy as np
import pytest

from harness import CUDA_TYPE, DeviceBuffer, N, T
from oracle import pyoracle as orc
from vulkanizer_b200 import capi

C_GELU = 0.7978845608


def gelu(x):
    return 0.5 * x * (1.0 + np.tanh(C_GELU * (x + 0.044715 * x ** 3)))


def gelu_grad(x):
    t = np.tanh(C_GELU * (x + 0.044715 * x ** 3))
    return 0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * C_GELU * (1.0 + 3 * 0.044715 * x * x)


def round_to(x, kind):
    if kind == "f32":
        return x.astype(np.float32).astype(np.float64)
    return orc.to_float(orc.to_storage(x.astype(np.float32), kind), kind).astype(np.float64)


@pytest.fixture(scope="module")
def lt(cuda):
    handle = capi.CublasLt()
    yield handle
    handle.destroy()


class Problem:
    """Operands of one TN or NN product in column order, their fp64 values, and alpha * op(A) op(B) + beta * C in fp64."""

    def __init__(self, cuda, ta, m, n, k, kind, alpha, beta, seed):
        self.ta, self.m, self.n, self.k, self.kind, self.alpha, self.beta = ta, m, n, k, kind, alpha, beta
        self.rows_a, cols_a = (k, m) if ta == T else (m, k)
        A, av = orc.fill_lcg(kind, self.rows_a * cols_a, seed)
        B, bv = orc.fill_lcg(kind, k * n, seed + 1)
        Cm, cv = orc.fill_lcg(kind, m * n, seed + 2)
        bias, biasv = orc.fill_lcg(kind, max(m, n), seed + 3)
        a = av.astype(np.float64).reshape(cols_a, self.rows_a).T       # stored matrix, rows x cols
        self.opa = a.T if ta == T else a                              # m x k
        self.b = bv.astype(np.float64).reshape(n, k).T                # k x n
        self.c = cv.astype(np.float64).reshape(n, m).T
        self.bias = biasv.astype(np.float64)
        self.y = alpha * (self.opa @ self.b) + beta * self.c           # m x n
        self.dA, self.dB, self.dC, self.dBias = (DeviceBuffer(cuda, x) for x in (A, B, Cm, bias))
        self.t = CUDA_TYPE[kind]
        self.tol_rel = (1e-5 if kind == "f32" else 4e-3 if kind == "f16" else 1.6e-2) * math.sqrt(k)

    def run(self, lt, dD, **kw):
        lt.matmul(self.ta, N, self.m, self.n, self.k, self.alpha, self.dA.ptr, self.t, self.rows_a, self.dB.ptr, self.t, self.k, self.beta,
                  self.dC.ptr, self.t, self.m, dD.ptr, self.t, self.m, **kw)

    def close(self, got, want):
        return np.abs(got - want) <= self.tol_rel * np.maximum(1.0, np.abs(want))


SHAPES = [("generic f16 unaligned", T, 70, 33, 33, "f16", capi.PATH_GENERIC), ("sgemm", N, 130, 50, 64, "f32", capi.PATH_SGEMM),
          ("tcgen05 f16", T, 256, 136, 128, "f16", capi.PATH_UMMA), ("tcgen05 bf16 ragged", T, 200, 72, 192, "bf16", capi.PATH_UMMA)]


@pytest.mark.gpu
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: s[0])
def test_relu_aux_then_drelu_bgrad(cuda, lt, shape):
    _, ta, m, n, k, kind, path = shape
    p = Problem(cuda, ta, m, n, k, kind, 1.0, 0.5, 41)
    aux_ld = (m + 127) // 128 * 128
    mask0 = np.full(aux_ld * n // 8, 0xA5, dtype=np.uint8)   # stale bits that the call must overwrite
    dMask, dD = DeviceBuffer(cuda, mask0), DeviceBuffer(cuda, orc.to_storage(np.zeros(m * n, dtype=np.float32), kind))
    p.run(lt, dD, epilogue=capi.LT_EPILOGUE_RELU_AUX_BIAS, bias=p.dBias.ptr, aux=dMask.ptr, aux_ld=aux_ld)
    assert lt.last_path() == path
    x = round_to(p.y, kind) + p.bias[:m, None]                 # D is rounded once before the bias, as for the reference's epilogues
    got = orc.to_float(dD.download(), kind).astype(np.float64).reshape(n, m).T
    assert p.close(got, np.maximum(x, 0.0)).all()
    bits = np.unpackbits(dMask.download(), bitorder="little").reshape(n, aux_ld).T[:m]   # bit row + col * aux_ld
    sure = np.abs(x) > p.tol_rel * np.maximum(1.0, np.abs(x))  # where rounding cannot flip the sign
    assert (bits[sure] == (x[sure] > 0)).all()

    # backward: D = (alpha A B + beta C) masked by the forward bits; bias = row sums of the stored D
    dG, dGrad = DeviceBuffer(cuda, orc.to_storage(np.zeros(m * n, dtype=np.float32), kind)), DeviceBuffer(cuda, orc.to_storage(np.zeros(m, dtype=np.float32), kind))
    p.run(lt, dG, epilogue=capi.LT_EPILOGUE_DRELU_BGRAD, bias=dGrad.ptr, aux=dMask.ptr, aux_ld=aux_ld)
    g = orc.to_float(dG.download(), kind).astype(np.float64).reshape(n, m).T
    assert p.close(g, p.y * bits).all()
    sums = orc.to_float(dGrad.download(), kind).astype(np.float64)
    want = g.sum(axis=1)
    assert (np.abs(sums - want) <= p.tol_rel * math.sqrt(n) * np.maximum(1.0, np.abs(want))).all()


@pytest.mark.gpu
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: s[0])
def test_gelu_aux_then_dgelu(cuda, lt, shape):
    _, ta, m, n, k, kind, path = shape
    p = Problem(cuda, ta, m, n, k, kind, 0.5, 0.0, 51)
    aux_ld = m + 8
    zeros = orc.to_storage(np.zeros(aux_ld * n, dtype=np.float32), kind)
    dAux, dD = DeviceBuffer(cuda, zeros), DeviceBuffer(cuda, zeros[:m * n].copy())
    p.run(lt, dD, epilogue=capi.LT_EPILOGUE_GELU_AUX_BIAS, bias=p.dBias.ptr, aux=dAux.ptr, aux_ld=aux_ld)
    assert lt.last_path() == path
    x = round_to(p.y, kind) + p.bias[:m, None]
    aux = orc.to_float(dAux.download(), kind).astype(np.float64).reshape(n, aux_ld).T
    assert p.close(aux[:m], x).all() and (aux[m:] == 0).all()
    got = orc.to_float(dD.download(), kind).astype(np.float64).reshape(n, m).T
    assert p.close(got, gelu(x)).all()
    dG = DeviceBuffer(cuda, zeros[:m * n].copy())
    p.run(lt, dG, epilogue=capi.LT_EPILOGUE_DGELU, aux=dAux.ptr, aux_ld=aux_ld)
    g = orc.to_float(dG.download(), kind).astype(np.float64).reshape(n, m).T
    assert p.close(g, p.y * gelu_grad(aux[:m])).all()


@pytest.mark.gpu
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: s[0])
def test_operand_bias_gradients(cuda, lt, shape):
    _, ta, m, n, k, kind, _ = shape
    p = Problem(cuda, ta, m, n, k, kind, 1.0, 0.0, 61)
    zeros = orc.to_storage(np.zeros(m * n, dtype=np.float32), kind)
    for epilogue, want in ((capi.LT_EPILOGUE_BGRADA, p.opa.sum(axis=1)), (capi.LT_EPILOGUE_BGRADB, p.b.sum(axis=0))):
        dD, dGrad = DeviceBuffer(cuda, zeros.copy()), DeviceBuffer(cuda, np.zeros(len(want), dtype=np.float32))
        p.run(lt, dD, epilogue=epilogue, bias=dGrad.ptr, bias_type=capi.CUDA_R_32F)
        assert p.close(orc.to_float(dD.download(), kind).astype(np.float64).reshape(n, m).T, p.y).all()
        assert np.allclose(dGrad.download(), want, rtol=1e-5 * math.sqrt(k), atol=1e-5 * math.sqrt(k))


@pytest.mark.gpu
@pytest.mark.parametrize("kind, m, n, k", [("f32", 45, 70, 33), ("f16", 136, 256, 128)])
@pytest.mark.parametrize("orders", [(1, 1, 1, 1), (1, 0, 0, 0), (0, 1, 1, 1)], ids=["all rows", "A in row order", "B, C, D in row order"])
def test_row_order_layouts(cuda, lt, kind, m, n, k, orders):
    """D = relu(alpha A B + beta C + bias) with some matrices stored row-major (no transposes requested): a row-order matrix of
    r x c with pitch ld is the c x r column-order matrix with the same ld, and a row-order D is computed as D^T."""
    oa, ob, oc, od = orders
    rng_a, av = orc.fill_lcg(kind, m * k, 71)
    rng_b, bv = orc.fill_lcg(kind, k * n, 72)
    rng_c, cv = orc.fill_lcg(kind, m * n, 73)
    bias, biasv = orc.fill_lcg(kind, m, 74)

    def matrix(values, rows, cols, order):
        v = values.astype(np.float64)
        return v.reshape(rows, cols) if order == 1 else v.reshape(cols, rows).T

    a, b, c = matrix(av, m, k, oa), matrix(bv, k, n, ob), matrix(cv, m, n, oc)
    x = round_to(0.5 * (a @ b) + 2.0 * c, kind) + biasv.astype(np.float64)[:, None]
    want = np.maximum(x, 0.0)
    dA, dB, dC, dBias = (DeviceBuffer(cuda, v) for v in (rng_a, rng_b, rng_c, bias))
    dD = DeviceBuffer(cuda, orc.to_storage(np.zeros(m * n, dtype=np.float32), kind))
    t = CUDA_TYPE[kind]
    ld = lambda rows, cols, order: cols if order == 1 else rows
    lt.matmul(N, N, m, n, k, 0.5, dA.ptr, t, ld(m, k, oa), dB.ptr, t, ld(k, n, ob), 2.0, dC.ptr, t, ld(m, n, oc), dD.ptr, t, ld(m, n, od),
              epilogue=capi.LT_EPILOGUE_RELU_BIAS, bias=dBias.ptr, order=orders)
    got = matrix(orc.to_float(dD.download(), kind), m, n, od)
    rel = (1e-5 if kind == "f32" else 4e-3) * math.sqrt(k)
    assert (np.abs(got - want) <= rel * np.maximum(1.0, np.abs(want))).all()
    if kind == "f16":
        assert lt.last_path() == capi.PATH_UMMA
