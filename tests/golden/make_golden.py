"""Generates tests/golden/cpu_gemm_golden.npz from k0zi/Vulkanizer's own CPU GEMM.

Run in a checkout that has the Vulkanizer tree (oracle/Makefile compiles src/npu/{host,backend,route,detect}.cpp and
src/common/log.cpp from it into oracle/_ref/libvkref.so):

    make -C oracle && python tests/golden/make_golden.py

Each case stores its parameters and the bytes of C after `CpuBackend::gemm` (src/npu/backend.cpp:28-52); the inputs are
regenerated from the seeds by the LCG of the reference's acceptance test (tests/cublas.cpp:64-78), so the file stays small.
Also stored: every f16 -> f32 conversion and a sweep of f32 -> f16 / bf16 roundings from the reference's host.cpp.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import pyoracle as orc  # noqa: E402

CASES = [
    # ta, tb, m, n, k, batch, type a, b, c, alpha, beta
    (0, 0, 5, 4, 3, 2, "f32", "f32", "f32", 0.5, 2.0),
    (1, 0, 5, 4, 3, 2, "f16", "f16", "f16", 0.5, 2.0),
    (0, 1, 33, 17, 70, 1, "bf16", "bf16", "f32", 1.0, 0.0),
    (1, 1, 40, 31, 129, 3, "f16", "f32", "bf16", -1.25, 0.75),
    (1, 0, 64, 48, 256, 1, "f16", "f16", "f32", 1.0, 0.5),
    (0, 0, 70, 33, 129, 1, "f32", "f32", "f32", 1.0, 0.0),
    (1, 0, 130, 1, 1000, 1, "f32", "f32", "f32", 0.5, -2.0),
    (0, 0, 1, 90, 77, 2, "bf16", "bf16", "bf16", 1.0, 1.0),
]


def shapes(ta, tb, m, n, k):
    rows_a, cols_a = (k, m) if ta else (m, k)
    rows_b, cols_b = (n, k) if tb else (k, n)
    return rows_a + 3, cols_a, rows_b + 1, cols_b, m + 2


def inputs(case):
    ta, tb, m, n, k, batch, ka, kb, kc, alpha, beta = case
    lda, cols_a, ldb, cols_b, ldc = shapes(ta, tb, m, n, k)
    A, _ = orc.fill_lcg(ka, lda * cols_a * batch, 1)
    B, _ = orc.fill_lcg(kb, ldb * cols_b * batch, 2)
    C, _ = orc.fill_lcg(kc, ldc * n * batch, 3)
    return A, B, C, (lda, lda * cols_a, ldb, ldb * cols_b, ldc, ldc * n)


def main():
    ref = orc.reference()
    assert ref is not None, "oracle/_ref/libvkref.so is missing: run `make -C oracle` with the Vulkanizer tree present"
    out = {}
    for i, case in enumerate(CASES):
        ta, tb, m, n, k, batch, ka, kb, kc, alpha, beta = case
        A, B, C, (lda, sa, ldb, sb, ldc, sc) = inputs(case)
        got = orc.gemm_f32(ta, tb, m, n, k, batch, alpha, A, ka, lda, sa, B, kb, ldb, sb, beta, C.copy(), kc, ldc, sc, use_reference=True)
        out[f"case{i}"] = np.frombuffer(got.tobytes(), dtype=np.uint8)
    out["half_to_float"] = np.array([ref.vkref_half_to_float(h) for h in range(65536)], dtype=np.float32).view(np.uint32)
    rng = np.random.default_rng(7)
    sweep = (rng.standard_normal(4096) * np.float32(10.0) ** rng.integers(-9, 6, 4096)).astype(np.float32)
    sweep = np.concatenate([sweep, np.array([65520.0, 1 + 1 / 2048, 2.9802322e-08, 1 + 1 / 256, 0.0, -0.0, 65504.0, 6.1035156e-05,
                                             5.9604645e-08, np.inf, -np.inf], dtype=np.float32)])
    out["round_inputs"] = sweep
    out["to_half"] = np.array([ref.vkref_float_to_half(float(v)) for v in sweep], dtype=np.uint16)
    out["to_bf16"] = np.array([ref.vkref_float_to_bf16(float(v)) for v in sweep], dtype=np.uint16)
    np.savez_compressed(Path(__file__).with_name("cpu_gemm_golden.npz"), **out)
    print("wrote", Path(__file__).with_name("cpu_gemm_golden.npz"))


if __name__ == "__main__":
    main()
