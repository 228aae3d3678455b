"""Test harness: device buffers (torch, for memory only), the reference acceptance test's data and tolerance,
and one function that runs a GEMM case through the C ABI and returns what the checks need.

The data, padding of leading dimensions and tolerance follow k0zi/Vulkanizer's tests/cublas.cpp:64-78, :113-117
and :174-181, so a case here reads like a row of its case table (:598-682).
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import numpy as np

from oracle import pyoracle as orc
from vulkanizer_b200 import capi

CUDA_TYPE = {"f32": capi.CUDA_R_32F, "f16": capi.CUDA_R_16F, "bf16": capi.CUDA_R_16BF, "s8": capi.CUDA_R_8I,
             "s32": capi.CUDA_R_32I, "f64": capi.CUDA_R_64F}
ELEM = {"f32": 4, "f16": 2, "bf16": 2, "s8": 1, "s32": 4, "f64": 8}
N, T = capi.OP_N, capi.OP_T


class DeviceBuffer:
    """Device memory holding a numpy array's bytes, with poisoned guard bands before and after."""
    GUARD = 256

    def __init__(self, torch, host: np.ndarray):
        self.torch = torch
        self.host_dtype = host.dtype
        self.count = host.size
        raw = np.frombuffer(host.tobytes(), dtype=np.uint8)
        self.nbytes = raw.size
        padded = np.full(self.nbytes + 2 * self.GUARD, 0xA5, dtype=np.uint8)
        padded[self.GUARD:self.GUARD + self.nbytes] = raw
        self.t = torch.from_numpy(padded).cuda()
        self.ptr = self.t.data_ptr() + self.GUARD

    def download(self) -> np.ndarray:
        self.torch.cuda.synchronize()
        raw = self.t.cpu().numpy()
        assert (raw[:self.GUARD] == 0xA5).all() and (raw[self.GUARD + self.nbytes:] == 0xA5).all(), "write outside the buffer"
        return np.frombuffer(raw[self.GUARD:self.GUARD + self.nbytes].tobytes(), dtype=self.host_dtype).copy()


@dataclass
class Case:
    name: str
    ta: int
    tb: int
    m: int
    n: int
    k: int
    type_a: str
    type_b: str
    type_c: str
    alpha: float
    beta: float
    batch: int = 1          # > 1 strided batch; < -1 pointer-array batch of -batch entries
    compute: int = capi.COMPUTE_32F
    aligned: bool = False   # leading dimensions rounded up to multiples of 8

    def __str__(self):
        return self.name


def layout(c: Case):
    batch = abs(c.batch)
    rows_a, cols_a = (c.m, c.k) if c.ta == N else (c.k, c.m)
    rows_b, cols_b = (c.k, c.n) if c.tb == N else (c.n, c.k)
    pad = (lambda rows, extra: (rows + extra + 7) // 8 * 8) if c.aligned else (lambda rows, extra: rows + extra)
    lda, ldb, ldc = pad(rows_a, 3), pad(rows_b, 1), c.m + 2
    return batch, lda, ldb, ldc, lda * cols_a, ldb * cols_b, ldc * c.n


def tolerance(c: Case, want: np.ndarray, want_abs: np.ndarray) -> np.ndarray:
    """tests/cublas.cpp:174-181."""
    rel = 1e-5 if c.type_c == "f32" else 2e-3 if c.type_c == "f16" else 1.6e-2
    tol = rel * np.maximum(1.0, np.abs(want)) * math.sqrt(c.k + 1.0)
    if c.compute in (capi.COMPUTE_16F, capi.COMPUTE_32F_FAST_16F):
        tol = tol + want_abs * 2.0 ** -10
    return tol


def run_case(torch, blas: capi.Cublas, c: Case):
    """Runs the case through the C ABI. Returns (got, want, tol, c_before, path) as float arrays over C's storage."""
    batch, lda, ldb, ldc, sA, sB, sC = layout(c)
    A, _ = orc.fill_lcg(c.type_a, sA * batch, 1)
    B, _ = orc.fill_lcg(c.type_b, sB * batch, 2)
    Cm, c_values = orc.fill_lcg(c.type_c, sC * batch, 3)
    want, want_abs = orc.gemm_fp64(c.ta != N, c.tb != N, c.m, c.n, c.k, batch, c.alpha, A, c.type_a, lda, sA, B, c.type_b, ldb, sB,
                                   c.beta, Cm, c.type_c, ldc, sC)
    dA, dB, dC = DeviceBuffer(torch, A), DeviceBuffer(torch, B), DeviceBuffer(torch, Cm)
    ta, tb, tc = CUDA_TYPE[c.type_a], CUDA_TYPE[c.type_b], CUDA_TYPE[c.type_c]
    plain = c.type_a == c.type_b == c.type_c == "f32"
    if c.batch == 1 and plain:
        blas.sgemm(c.ta, c.tb, c.m, c.n, c.k, c.alpha, dA.ptr, lda, dB.ptr, ldb, c.beta, dC.ptr, ldc)
    elif c.batch == 1:
        blas.gemm_ex(c.ta, c.tb, c.m, c.n, c.k, c.alpha, dA.ptr, ta, lda, dB.ptr, tb, ldb, c.beta, dC.ptr, tc, ldc, c.compute,
                     capi.GEMM_DEFAULT_TENSOR_OP)
    elif c.batch > 1:
        blas.gemm_strided_batched_ex(c.ta, c.tb, c.m, c.n, c.k, c.alpha, dA.ptr, ta, lda, sA, dB.ptr, tb, ldb, sB, c.beta, dC.ptr,
                                     tc, ldc, sC, batch, c.compute)
    else:
        ptrs = np.array([dA.ptr + b * sA * ELEM[c.type_a] for b in range(batch)] +
                        [dB.ptr + b * sB * ELEM[c.type_b] for b in range(batch)] +
                        [dC.ptr + b * sC * ELEM[c.type_c] for b in range(batch)], dtype=np.uint64)
        dP = DeviceBuffer(torch, ptrs)
        blas.gemm_batched_ex(c.ta, c.tb, c.m, c.n, c.k, c.alpha, dP.ptr, ta, lda, dP.ptr + 8 * batch, tb, ldb, c.beta,
                             dP.ptr + 16 * batch, tc, ldc, batch, capi.COMPUTE_32F)
        torch.cuda.synchronize()
    path = blas.last_path()
    got = orc.to_float(dC.download(), c.type_c)
    return got, want, tolerance(c, want, want_abs), c_values, path
