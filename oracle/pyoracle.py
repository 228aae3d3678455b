"""TEST INFRASTRUCTURE, NOT PRODUCT CODE: ctypes access to the CPU checker.

``liboracle.so`` is the C restatement in oracle/oracle.c; ``libvkref.so`` is k0zi/Vulkanizer's own CPU GEMM
(src/npu/backend.cpp:28-52, src/npu/host.cpp:209-235) compiled from its sources by oracle/Makefile. Only tests/,
the smoke test and the benchmark's CPU-baseline / reference arm may import this module.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
TYPE_CODE = {"f32": 0, "f16": 1, "bf16": 2, "s8": 3}
_i, _ll, _f, _vp = C.c_int, C.c_int64, C.c_float, C.c_void_p


def build() -> None:
    subprocess.run(["make", "-C", str(HERE), "all"], check=True)


_oracle = None
_ref = None


def oracle() -> C.CDLL:
    global _oracle
    if _oracle is None:
        path = HERE / "_build" / "liboracle.so"
        if not path.exists():
            build()
        lib = C.CDLL(str(path))
        lib.oracle_half_to_float.argtypes, lib.oracle_half_to_float.restype = [C.c_uint16], _f
        lib.oracle_float_to_half.argtypes, lib.oracle_float_to_half.restype = [_f], C.c_uint16
        lib.oracle_bf16_to_float.argtypes, lib.oracle_bf16_to_float.restype = [C.c_uint16], _f
        lib.oracle_float_to_bf16.argtypes, lib.oracle_float_to_bf16.restype = [_f], C.c_uint16
        lib.oracle_fill_lcg.argtypes, lib.oracle_fill_lcg.restype = [_i, _ll, C.c_uint32, _vp, _vp], None
        gemm = [_i, _i, _ll, _ll, _ll, _ll, _f, _vp, _i, _ll, _ll, _vp, _i, _ll, _ll, _f, _vp, _i, _ll, _ll]
        lib.oracle_gemm_f32.argtypes, lib.oracle_gemm_f32.restype = gemm, None
        lib.oracle_gemm_fp64.argtypes, lib.oracle_gemm_fp64.restype = gemm + [_vp, _vp], None
        lib.oracle_dots_fp64.argtypes = [_i, _i, _ll, _vp, _i, _ll, _vp, _i, _ll, _vp, _ll, _vp, _ll, _vp]
        lib.oracle_dots_fp64.restype = None
        lib.oracle_lt_fp64.argtypes = [_i, _i, _ll, _ll, _ll, _ll, _f, _vp, _vp, _f, _vp, _vp, _i, _i, _vp]
        lib.oracle_lt_fp64.restype = None
        lib.oracle_gemm_s8.argtypes = [_i, _i, _ll, _ll, _ll, _ll, C.c_int32, _vp, _ll, _ll, _vp, _ll, _ll, C.c_int32, _vp, _ll, _ll]
        lib.oracle_gemm_s8.restype = None
        _oracle = lib
    return _oracle


def reference():
    """The reference's own CPU GEMM, or None when oracle/_ref/libvkref.so was not built."""
    global _ref
    if _ref is None:
        path = HERE / "_ref" / "libvkref.so"
        if not path.exists():
            return None
        lib = C.CDLL(str(path))
        lib.vkref_cpu_gemm.argtypes = [_i, _i, _ll, _ll, _ll, _ll, _f, _vp, _i, _ll, _ll, _vp, _i, _ll, _ll, _f, _vp, _i, _ll, _ll]
        lib.vkref_cpu_gemm.restype = _i
        lib.vkref_staged_gemm.argtypes = [_i, _i, _ll, _ll, _ll, _f, _vp, _i, _ll, _vp, _i, _ll, _f, _vp, _i, _ll]
        lib.vkref_staged_gemm.restype = _i
        lib.vkref_float_to_half.argtypes, lib.vkref_float_to_half.restype = [_f], C.c_uint16
        lib.vkref_half_to_float.argtypes, lib.vkref_half_to_float.restype = [C.c_uint16], _f
        lib.vkref_float_to_bf16.argtypes, lib.vkref_float_to_bf16.restype = [_f], C.c_uint16
        lib.vkref_bf16_to_float.argtypes, lib.vkref_bf16_to_float.restype = [C.c_uint16], _f
        lib.vkref_hardware_threads.argtypes, lib.vkref_hardware_threads.restype = [], _i
        _ref = lib
    return _ref


def _ptr(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


# ---- storage helpers: matrices travel as raw numpy buffers (uint16 for f16 / bf16) ----

def storage_dtype(kind: str):
    return {"f32": np.float32, "f16": np.uint16, "bf16": np.uint16, "s8": np.int8, "s32": np.int32, "f64": np.float64}[kind]


def to_storage(values: np.ndarray, kind: str) -> np.ndarray:
    """float32 values -> storage bits of `kind` (round to nearest even, numpy's conversions)."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    if kind == "f32":
        return v.copy()
    if kind == "f16":
        return v.astype(np.float16).view(np.uint16)
    if kind == "bf16":
        u = v.view(np.uint32).astype(np.uint64)
        rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
        return rounded.astype(np.uint16)
    raise ValueError(kind)


def to_float(bits: np.ndarray, kind: str) -> np.ndarray:
    if kind == "f32":
        return np.asarray(bits, dtype=np.float32)
    if kind == "f16":
        return bits.view(np.float16).astype(np.float32)
    if kind == "bf16":
        return (bits.astype(np.uint32) << 16).view(np.float32)
    return bits.astype(np.float32)


def fill_lcg(kind: str, count: int, seed: int):
    """Data of the reference's acceptance test (tests/cublas.cpp:64-78): storage bits and the floats they hold."""
    bits = np.zeros(max(count, 1), dtype=storage_dtype(kind))[:count]
    bits = np.ascontiguousarray(bits)
    values = np.zeros(count, dtype=np.float32)
    if count:
        oracle().oracle_fill_lcg(TYPE_CODE[kind], count, seed, _ptr(bits), _ptr(values))
    return bits, values


def gemm_f32(ta, tb, m, n, k, batch, alpha, A, kind_a, lda, stride_a, B, kind_b, ldb, stride_b, beta, Cm, kind_c, ldc, stride_c,
             use_reference=False):
    """C (modified in place and returned) by the restated reference CPU GEMM, or by the reference itself."""
    args = (int(ta), int(tb), m, n, k, batch, alpha, _ptr(A), TYPE_CODE[kind_a], lda, stride_a, _ptr(B), TYPE_CODE[kind_b], ldb,
            stride_b, beta, _ptr(Cm), TYPE_CODE[kind_c], ldc, stride_c)
    if use_reference:
        assert reference().vkref_cpu_gemm(*args) == 1
    else:
        oracle().oracle_gemm_f32(*args)
    return Cm


def gemm_fp64(ta, tb, m, n, k, batch, alpha, A, kind_a, lda, stride_a, B, kind_b, ldb, stride_b, beta, Cm, kind_c, ldc, stride_c):
    """(want, wantAbs) as float32 arrays shaped like C's storage, per tests/cublas.cpp:121-136."""
    want = np.zeros(Cm.size, dtype=np.float32)
    want_abs = np.zeros(Cm.size, dtype=np.float32)
    oracle().oracle_gemm_fp64(int(ta), int(tb), m, n, k, batch, alpha, _ptr(A), TYPE_CODE[kind_a], lda, stride_a, _ptr(B),
                              TYPE_CODE[kind_b], ldb, stride_b, beta, _ptr(Cm), TYPE_CODE[kind_c], ldc, stride_c, _ptr(want),
                              _ptr(want_abs))
    return want, want_abs


def dots_fp64(ta, tb, k, A, kind_a, lda, B, kind_b, ldb, rows, cols):
    rows = np.ascontiguousarray(rows, dtype=np.int64)
    cols = np.ascontiguousarray(cols, dtype=np.int64)
    out = np.zeros((len(cols), len(rows)), dtype=np.float64)  # column-major (rows fastest)
    oracle().oracle_dots_fp64(int(ta), int(tb), k, _ptr(A), TYPE_CODE[kind_a], lda, _ptr(B), TYPE_CODE[kind_b], ldb, _ptr(rows),
                              len(rows), _ptr(cols), len(cols), _ptr(out))
    return out.T  # [row, col]


def lt_fp64(ta, tb, m, n, k, batch, alpha, A, B, beta, Cm, bias, kind, epilogue_bits):
    want = np.zeros(m * n * batch, dtype=np.float32)
    oracle().oracle_lt_fp64(int(ta), int(tb), m, n, k, batch, alpha, _ptr(A), _ptr(B), beta, _ptr(Cm),
                            _ptr(bias) if bias is not None else None, TYPE_CODE[kind], epilogue_bits, _ptr(want))
    return want


def gemm_s8(ta, tb, m, n, k, batch, alpha, A, lda, stride_a, B, ldb, stride_b, beta, Cm, ldc, stride_c):
    oracle().oracle_gemm_s8(int(ta), int(tb), m, n, k, batch, int(alpha), _ptr(A), lda, stride_a, _ptr(B), ldb, stride_b, int(beta),
                            _ptr(Cm), ldc, stride_c)
    return Cm


def attention_fp64(q, k, v, scale, mask):
    """softmax(scale q k^T + mask) v and its logsumexp in fp64, as the reference's own test computes what it expects
    (tests/attention.cpp:190-228): q is [batches, heads, numQ, dim], k and v [batches, kvHeads, numK, dim]; query head h reads
    head h // (heads // kvHeads); mask 1 hides key j from query i when j > i, mask 2 when j > i + numK - numQ; a row that sees
    no key gives zeros and a logsumexp of 0."""
    q, k, v = (np.asarray(x, dtype=np.float64) for x in (q, k, v))
    batches, heads, num_q, _ = q.shape
    kv_heads, num_k = k.shape[1], k.shape[2]
    group = heads // kv_heads
    out = np.zeros(q.shape[:3] + (v.shape[3],))
    lse = np.zeros(q.shape[:3])
    diag = num_k - num_q if mask == 2 else 0
    hidden = (np.arange(num_k)[None, :] > np.arange(num_q)[:, None] + diag) if mask else np.zeros((num_q, num_k), dtype=bool)
    for b in range(batches):
        for h in range(heads):
            s = scale * (q[b, h] @ k[b, h // group].T)
            s[hidden] = -np.inf
            mx = s.max(axis=1, initial=-np.inf)
            seen = np.isfinite(mx)
            e = np.where(np.isfinite(s), np.exp(s - np.where(seen, mx, 0.0)[:, None]), 0.0)
            total = e.sum(axis=1)
            out[b, h][seen] = (e @ v[b, h // group])[seen] / total[seen, None]
            lse[b, h][seen] = mx[seen] + np.log(total[seen])
    return out, lse
