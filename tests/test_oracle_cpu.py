"""The CPU checker itself: pinned against the reference's known answers, its compiled CPU GEMM and golden vectors.

Known answers: k0zi/Vulkanizer tests/npu.cpp:110-121 (conversions) and :125-169 (CPU GEMM against a direct column-major
loop, nothing outside the m x n window changes). Golden vectors: tests/golden/cpu_gemm_golden.npz, generated from the
reference's own CpuBackend::gemm by tests/golden/make_golden.py.
"""
import importlib.util
import math
from pathlib import Path

import numpy as np
import pytest

from oracle import pyoracle as orc

GOLDEN = Path(__file__).parent / "golden" / "cpu_gemm_golden.npz"
spec = importlib.util.spec_from_file_location("make_golden", Path(__file__).parent / "golden" / "make_golden.py")
make_golden = importlib.util.module_from_spec(spec)
spec.loader.exec_module(make_golden)


def test_conversion_known_answers():
    lib = orc.oracle()
    for v in [0.0, -0.0, 1.0, -2.5, 65504.0, 6.1035156e-05, 5.9604645e-08, 0.1, 3.14159]:
        assert abs(lib.oracle_half_to_float(lib.oracle_float_to_half(v)) - v) <= abs(v) * 1e-3
        assert abs(lib.oracle_bf16_to_float(lib.oracle_float_to_bf16(v)) - v) <= abs(v) * 8e-3
    assert lib.oracle_float_to_half(65520.0) == 0x7C00          # halfway past the largest half rounds to infinity
    assert lib.oracle_float_to_half(1.0 + 1.0 / 2048) == 0x3C00  # tie to even
    assert lib.oracle_float_to_half(2.9802322e-08) == 0          # half the smallest subnormal: tie to even
    assert lib.oracle_float_to_bf16(1.0 + 1.0 / 256) == 0x3F80   # tie to even
    assert math.isnan(lib.oracle_half_to_float(lib.oracle_float_to_half(float("nan"))))
    assert math.isnan(lib.oracle_bf16_to_float(lib.oracle_float_to_bf16(float("nan"))))


def test_conversions_match_golden():
    g = np.load(GOLDEN)
    lib = orc.oracle()
    got = np.array([lib.oracle_half_to_float(h) for h in range(65536)], dtype=np.float32).view(np.uint32)
    assert np.array_equal(got, g["half_to_float"])
    assert np.array_equal(np.array([lib.oracle_float_to_half(float(v)) for v in g["round_inputs"]], dtype=np.uint16), g["to_half"])
    assert np.array_equal(np.array([lib.oracle_float_to_bf16(float(v)) for v in g["round_inputs"]], dtype=np.uint16), g["to_bf16"])
    # numpy's own f32 -> f16 rounding agrees too (it is what the harness uses to make fp16 operands)
    finite = np.isfinite(g["round_inputs"])
    assert np.array_equal(g["round_inputs"][finite].astype(np.float16).view(np.uint16), g["to_half"][finite])
    assert np.array_equal(orc.to_storage(g["round_inputs"][finite], "bf16"), g["to_bf16"][finite])


@pytest.mark.parametrize("index", range(len(make_golden.CASES)))
def test_cpu_gemm_matches_golden_bit_for_bit(index):
    case = make_golden.CASES[index]
    ta, tb, m, n, k, batch, ka, kb, kc, alpha, beta = case
    A, B, C, (lda, sa, ldb, sb, ldc, sc) = make_golden.inputs(case)
    got = orc.gemm_f32(ta, tb, m, n, k, batch, alpha, A, ka, lda, sa, B, kb, ldb, sb, beta, C.copy(), kc, ldc, sc)
    want = np.load(GOLDEN)[f"case{index}"]
    assert np.array_equal(np.frombuffer(got.tobytes(), dtype=np.uint8), want)


@pytest.mark.parametrize("index", range(len(make_golden.CASES)))
def test_cpu_gemm_matches_compiled_reference(index):
    if orc.reference() is None:
        pytest.skip("oracle/_ref/libvkref.so not built (needs the Vulkanizer tree)")
    case = make_golden.CASES[index]
    ta, tb, m, n, k, batch, ka, kb, kc, alpha, beta = case
    A, B, C, (lda, sa, ldb, sb, ldc, sc) = make_golden.inputs(case)
    mine = orc.gemm_f32(ta, tb, m, n, k, batch, alpha, A, ka, lda, sa, B, kb, ldb, sb, beta, C.copy(), kc, ldc, sc)
    theirs = orc.gemm_f32(ta, tb, m, n, k, batch, alpha, A, ka, lda, sa, B, kb, ldb, sb, beta, C.copy(), kc, ldc, sc, use_reference=True)
    assert np.array_equal(mine, theirs)


@pytest.mark.parametrize("t", range(4))
@pytest.mark.parametrize("kind", ["f32", "f16"])
def test_cpu_gemm_against_direct_loop(t, kind):
    """tests/npu.cpp:125-169: m=5, n=4, k=3, batch 2, ld 7, alpha 0.5, beta 2; untouched outside the window."""
    ta, tb = bool(t & 1), bool(t & 2)
    m, n, k, batch, ld = 5, 4, 3, 2, 7
    stride = ld * 8
    idx = np.arange(stride * batch)
    A = orc.to_storage(((idx * 7) % 11 - 5).astype(np.float32), kind)
    B = orc.to_storage(((idx * 5) % 9 - 4).astype(np.float32), kind)
    C0 = orc.to_storage((idx % 3).astype(np.float32), kind)
    got = orc.to_float(orc.gemm_f32(ta, tb, m, n, k, batch, 0.5, A, kind, ld, stride, B, kind, ld, stride, 2.0, C0.copy(), kind, ld, stride), kind)
    a, b, c0 = orc.to_float(A, kind), orc.to_float(B, kind), orc.to_float(C0, kind)
    for bi in range(batch):
        for j in range(n):
            for i in range(m):
                s = sum(a[bi * stride + (p + i * ld if ta else i + p * ld)] * b[bi * stride + (j + p * ld if tb else p + j * ld)] for p in range(k))
                at = bi * stride + i + j * ld
                assert abs(got[at] - (0.5 * s + 2.0 * c0[at])) < 1e-3
    rows, cols = (idx % stride) % ld, (idx % stride) // ld
    outside = (rows >= m) | (cols >= n)
    assert np.array_equal(got[outside], c0[outside])


def test_fp64_reference_against_numpy():
    rng = np.random.default_rng(3)
    m, n, k = 37, 29, 53
    A = rng.standard_normal((k, m)).astype(np.float32)  # stored k x m column-major = op T
    B = rng.standard_normal((n, k)).astype(np.float32).T.copy()  # k x n
    C = rng.standard_normal((n, m)).astype(np.float32)
    # column-major buffers: a (rows, cols) column-major matrix is the transpose's C-order bytes
    a_cm = np.ascontiguousarray(A.T).ravel()      # k x m col-major <=> (m, k) C-order
    b_cm = np.ascontiguousarray(B.T).ravel()      # k x n col-major <=> (n, k) C-order
    c_cm = np.ascontiguousarray(C).ravel()        # m x n col-major <=> (n, m) C-order
    want, _ = orc.gemm_fp64(True, False, m, n, k, 1, 1.5, a_cm, "f32", k, 0, b_cm, "f32", k, 0, -0.5, c_cm, "f32", m, 0)
    ref = (1.5 * (A.T.astype(np.float64) @ B.astype(np.float64)) - 0.5 * C.T.astype(np.float64)).astype(np.float32)
    assert np.allclose(want.reshape(n, m).T, ref, rtol=0, atol=1e-6)


def test_int8_oracle_is_exact_integer_arithmetic():
    rng = np.random.default_rng(5)
    m, n, k = 19, 23, 301
    A = rng.integers(-127, 128, (m, k), dtype=np.int8)   # op T: stored k x m col-major <=> (m, k) C-order
    B = rng.integers(-127, 128, (n, k), dtype=np.int8)   # stored k x n col-major <=> (n, k) C-order
    C = rng.integers(-1000, 1000, (n, m), dtype=np.int32)
    got = orc.gemm_s8(True, False, m, n, k, 1, 3, A.ravel(), k, 0, B.ravel(), k, 0, -2, C.ravel().copy(), m, 0)
    ref = 3 * (A.astype(np.int64) @ B.astype(np.int64).T) - 2 * C.T
    assert np.array_equal(got.reshape(n, m).T, ref.astype(np.int32))
    sample = orc.dots_fp64(True, False, k, A.ravel(), "s8", k, B.ravel(), "s8", k, [0, 5, 18], [1, 22])
    assert np.array_equal(sample, (A.astype(np.int64) @ B.astype(np.int64).T)[[0, 5, 18]][:, [1, 22]].astype(np.float64))


def test_lcg_data_is_exact_in_every_storage_type():
    """tests/cublas.cpp:64-78: values are k / 64 with |k| <= 128, hence exact in f16, bf16 and TF32."""
    for kind in ("f32", "f16", "bf16"):
        bits, values = orc.fill_lcg(kind, 1000, 1)
        scaled = values * 64
        assert np.array_equal(scaled, np.round(scaled)) and np.abs(scaled).max() <= 128
        assert np.array_equal(orc.to_float(bits, kind), values)
    f32, _ = orc.fill_lcg("f32", 1000, 1)
    f16, _ = orc.fill_lcg("f16", 1000, 1)
    assert np.array_equal(f32, orc.to_float(f16, "f16"))


def test_synthetic_generators_are_deterministic_and_shaped():
    from vulkanizer_b200 import synth
    a = synth.normal(1, 100000, 0.02)
    assert np.array_equal(a[500:600], synth.normal(1, 100, 0.02, first=500))  # element i depends on (seed, i) only
    assert abs(float(a.mean())) < 3e-4 and abs(float(a.std()) - 0.02) < 3e-4
    u = synth.uniform(0, 100000)
    assert -1.0 <= u.min() and u.max() <= 1.0 and abs(float(u.mean())) < 0.01
    i8 = synth.int8_uniform(2, 100000)
    assert i8.min() == -127 and i8.max() == 127 and i8.dtype == np.int8
    assert not np.array_equal(synth.normal(1, 100), synth.normal(2, 100))


def test_synthetic_generator_has_the_same_values_on_a_torch_device():
    """The benchmark makes its largest operands with the torch form of vulkanizer_b200/synth.py (on the GPU); the checks
    regenerate samples with the numpy form. Both must give the same numbers: identical as bf16 / f16 storage, and as float32
    except where the math libraries' last fp64 bit flips a float32 rounding (far rarer than 1 in 10^5)."""
    import torch
    from vulkanizer_b200 import synth
    count, first = 1 << 18, (1 << 31) * 3 + 12345   # an offset beyond 32 bits, as the 32768 x 32768 operands have
    want = synth.normal(5, count, 0.02, first=first)
    got = synth.normal_torch(torch, 5, count, 0.02, first=first, device="cpu").numpy()
    assert (want == got).mean() > 0.99999
    assert np.array_equal(orc.to_storage(want, "bf16"), orc.to_storage(got, "bf16"))
    assert np.array_equal(orc.to_storage(want, "f16"), orc.to_storage(got, "f16"))
    out = torch.empty(1000, dtype=torch.bfloat16)
    synth.fill_normal_torch(torch, out, 5, 1.0, first=77, block=256)
    assert np.array_equal(out.view(torch.int16).numpy().view(np.uint16), orc.to_storage(synth.normal(5, 1000, 1.0, first=77), "bf16"))


def test_attention_oracle_against_plain_loops():
    """attention_fp64 against the loop form of the reference's own expected-value computation (tests/attention.cpp:190-228) on a
    case small enough for pure Python: both masks, grouped heads, a row that sees no key."""
    rng = np.random.default_rng(3)
    batches, heads, kv_heads, num_q, num_k, dim = 1, 2, 1, 5, 3, 4
    q, k, v = rng.standard_normal((batches, heads, num_q, dim)), rng.standard_normal((batches, kv_heads, num_k, dim)), rng.standard_normal((batches, kv_heads, num_k, dim))
    for mask in (0, 1, 2):
        out, lse = orc.attention_fp64(q, k, v, 0.5, mask)
        diag = num_k - num_q if mask == 2 else 0
        for h in range(heads):
            for i in range(num_q):
                s = [0.5 * float(q[0, h, i] @ k[0, 0, j]) if not (mask and j > i + diag) else -math.inf for j in range(num_k)]
                mx = max(s)
                e = [0.0 if math.isinf(x) else math.exp(x - mx) for x in s]
                total = sum(e)
                want = sum(e[j] * v[0, 0, j] for j in range(num_k)) / total if total else np.zeros(dim)
                assert np.allclose(out[0, h, i], want, rtol=1e-12, atol=1e-12)
                assert abs(lse[0, h, i] - (mx + math.log(total) if total else 0.0)) < 1e-12
