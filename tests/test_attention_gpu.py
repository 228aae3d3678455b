"""vkzbAttentionForward (include/vkzb_attention.h): softmax(scale Q K^T + mask) V in one tcgen05 kernel.

The expected values are the fp64 computation of the reference's attention test (tests/attention.cpp:190-228, restated in
oracle/pyoracle.py), held to that test's tolerances (tests/attention.cpp:187: 6e-3 for f16, 4e-2 for bf16, relative to
1 + |expected|; logsumexp within 1e-3). The cases follow that test's list: both 16-bit types, both masks, grouped-query heads,
logsumexp, lengths that are not multiples of the tile, strides with padding, and [batch, sequence, head, dim] tensors.
"""
import math

import numpy as np
import pytest

from harness import CUDA_TYPE, DeviceBuffer
from oracle import pyoracle as orc
from vulkanizer_b200 import capi


def padded(values, row_pitch):
    """[..., rows, dim] -> flat storage with `row_pitch` elements per row (the padding holds 7.0, which must never be read)."""
    out = np.full(values.shape[:-1] + (row_pitch,), 7.0, dtype=np.float32)
    out[..., :values.shape[-1]] = values
    return out


def run_case(cuda, kind, batches, heads, kv_heads, num_q, num_k, dim, mask, scale, pad=0, lse=False, interleaved=False, seed=5):
    lib = capi.cublas_library()
    _, qv = orc.fill_lcg(kind, batches * heads * num_q * dim, seed)
    _, kv = orc.fill_lcg(kind, batches * kv_heads * num_k * dim, seed + 1)
    _, vv = orc.fill_lcg(kind, batches * kv_heads * num_k * dim, seed + 2)
    q = qv.reshape(batches, heads, num_q, dim)
    k = kv.reshape(batches, kv_heads, num_k, dim)
    v = vv.reshape(batches, kv_heads, num_k, dim)
    want, want_lse = orc.attention_fp64(q, k, v, scale, mask)

    def lay_out(x):
        """-> (flat fp32 values as stored, (row, head, batch) strides in elements)"""
        b, h, n, _ = x.shape
        if interleaved:  # [batch, sequence, head, dim]
            pitch = dim + pad
            stored = padded(x.transpose(0, 2, 1, 3), pitch)
            return stored.reshape(-1), (h * pitch, pitch, n * h * pitch)
        pitch = dim + pad
        stored = padded(x, pitch)  # [batch, head, sequence, pitch]
        return stored.reshape(-1), (pitch, n * pitch, h * n * pitch)

    (qs, q_str), (ks, k_str), (vs, v_str) = lay_out(q), lay_out(k), lay_out(v)
    o_host, o_str = lay_out(np.zeros_like(want, dtype=np.float32))
    dQ, dK, dV = (DeviceBuffer(cuda, orc.to_storage(x, kind)) for x in (qs, ks, vs))
    dO = DeviceBuffer(cuda, orc.to_storage(np.full(o_host.size, 3.0, dtype=np.float32), kind))
    dL = DeviceBuffer(cuda, np.full(batches * heads * num_q, 9.0, dtype=np.float32)) if lse else None
    status = capi.attention_forward(None, CUDA_TYPE[kind], batches, heads, kv_heads, num_q, num_k, dim, mask, scale, dQ.ptr, q_str, dK.ptr, k_str,
                                    dV.ptr, v_str, dO.ptr, o_str, dL.ptr if lse else None)
    assert status == capi.STATUS_SUCCESS
    got_flat = orc.to_float(dO.download(), kind).astype(np.float64)
    assert lib.vkzbAttentionStatus() == 0
    pitch = dim + pad
    if interleaved:
        got_all = got_flat.reshape(batches, num_q, heads, pitch).transpose(0, 2, 1, 3)
    else:
        got_all = got_flat.reshape(batches, heads, num_q, pitch)
    got = got_all[..., :dim]
    if pad:
        assert (got_all[..., dim:] == 3.0).all(), "the padding of O was written"
    tol = 6e-3 if kind == "f16" else 4e-2
    err = np.abs(got - want) / (1.0 + np.abs(want))
    assert err.max() <= tol, f"largest error {err.max():.2e} at {np.unravel_index(err.argmax(), err.shape)}"
    if lse:
        got_lse = dL.download().astype(np.float64).reshape(batches, heads, num_q)
        assert np.abs(got_lse - want_lse).max() <= 1e-3
    return err.max()


CASES = [
    # name, type, batches, heads, kvHeads, numQ, numK, dim, mask, scale, keyword arguments
    ("one tile f16 d128", "f16", 1, 1, 1, 128, 128, 128, 0, 1 / math.sqrt(128), {}),
    ("one tile f16 d64", "f16", 1, 1, 1, 128, 128, 64, 0, 0.125, {}),
    ("four key tiles, moving maximum", "f16", 1, 2, 2, 128, 512, 128, 0, 1.0, {"lse": True}),
    ("ragged lengths f16 d128", "f16", 2, 3, 3, 130, 200, 128, 0, 1 / math.sqrt(128), {"lse": True}),
    ("ragged lengths bf16 d64", "bf16", 2, 2, 2, 77, 333, 64, 0, 0.125, {}),
    ("causal from the top left", "f16", 1, 2, 2, 300, 300, 128, 1, 1 / math.sqrt(128), {"lse": True}),
    ("causal from the bottom right", "f16", 1, 2, 2, 130, 200, 128, 2, 1 / math.sqrt(128), {"lse": True}),
    ("bottom right with rows that see no key", "bf16", 1, 1, 1, 200, 130, 64, 2, 0.125, {"lse": True}),
    ("grouped-query heads", "bf16", 2, 4, 2, 150, 260, 128, 1, 1 / math.sqrt(128), {}),
    ("padded rows", "f16", 1, 2, 1, 140, 150, 64, 0, 0.125, {"pad": 8}),
    ("batch, sequence, head, dim tensors", "f16", 2, 4, 2, 160, 140, 128, 1, 1 / math.sqrt(128), {"interleaved": True, "lse": True}),
    ("a single query and key", "f16", 1, 1, 1, 1, 1, 64, 0, 1.0, {}),
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=lambda c: c[0])
def test_attention_matches_the_fp64_oracle(cuda, case):
    _, kind, batches, heads, kv_heads, num_q, num_k, dim, mask, scale, kw = case
    run_case(cuda, kind, batches, heads, kv_heads, num_q, num_k, dim, mask, scale, **kw)


@pytest.mark.gpu
def test_attention_over_the_batched_benchmark_shape(cuda):
    """A slice of the benchmark's batched-attention problem (heads of 1024 x 1024 x 128, f16): eight key tiles per query tile."""
    run_case(cuda, "f16", 1, 3, 3, 1024, 1024, 128, 0, 1 / math.sqrt(128), lse=True, seed=17)


@pytest.mark.gpu
def test_attention_refuses_what_it_cannot_serve(cuda):
    zeros = DeviceBuffer(cuda, np.zeros(4096, dtype=np.uint16))
    base = dict(stream=None, data_type=capi.CUDA_R_16F, batches=1, heads=1, kv_heads=1, num_q=8, num_k=8, head_dim=64, mask=0, scale=1.0,
                q=zeros.ptr, q_strides=(64, 512, 512), k=zeros.ptr, k_strides=(64, 512, 512), v=zeros.ptr, v_strides=(64, 512, 512),
                o=zeros.ptr, o_strides=(64, 512, 512))
    assert capi.attention_forward(**{**base, "head_dim": 96}) == capi.STATUS_NOT_SUPPORTED
    assert capi.attention_forward(**{**base, "data_type": capi.CUDA_R_32F}) == capi.STATUS_NOT_SUPPORTED
    assert capi.attention_forward(**{**base, "q_strides": (68, 512, 512)}) == capi.STATUS_NOT_SUPPORTED     # rows of 136 bytes
    assert capi.attention_forward(**{**base, "q": zeros.ptr + 2}) == capi.STATUS_NOT_SUPPORTED
    assert capi.attention_forward(**{**base, "kv_heads": 0}) == capi.STATUS_INVALID_VALUE
    assert capi.attention_forward(**{**base, "mask": 3}) == capi.STATUS_INVALID_VALUE
    assert capi.attention_forward(**{**base, "o": None}) == capi.STATUS_INVALID_VALUE
    assert capi.attention_forward(**{**base, "num_q": 0}) == capi.STATUS_SUCCESS
    assert (zeros.download() == 0).all()
