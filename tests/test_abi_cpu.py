"""The drop-in boundary without a GPU: the libraries load, export what include/*.h declares at NVIDIA's symbol version
nodes, agree with the CUDA toolkit's headers on every enum value they share, and answer the host-only calls as
k0zi/Vulkanizer's libraries do (src/cublas/cublas.cpp:699, 1028-1058; src/cublas/cublasLt.cpp:142-277; cublas_stubs.cpp:241-247).
No call here launches a kernel or needs a device.
"""
import ctypes as C
import re
import subprocess
from pathlib import Path

import pytest

import vulkanizer_b200 as vk
from vulkanizer_b200 import capi

ROOT = Path(__file__).resolve().parents[1]


def test_cublas_exports_every_declared_symbol():
    lib = vk.cublas_library()
    for name in vk.declared_symbols("vkzb_cublas.h") + vk.declared_symbols("vkzb_ext.h") + vk.declared_symbols("vkzb_attention.h"):
        assert hasattr(lib, name), name


def test_cublaslt_exports_every_declared_symbol():
    lib = vk.cublaslt_library()
    for name in vk.declared_symbols("vkzb_cublaslt.h"):
        if name.startswith("cublasLt"):
            assert hasattr(lib, name), name


def _dynamic_symbols(lib):
    out = subprocess.run(["nm", "-D", "--defined-only", str(vk.LIB_DIR / lib)], capture_output=True, text=True, check=True).stdout
    return [line.split()[-1] for line in out.splitlines() if line.strip()]


def test_symbol_version_nodes_match_nvidia():
    syms = _dynamic_symbols("libcublas.so.12")
    assert "cublasGemmEx@@libcublas.so.12" in syms and "cublasSgemm_v2@@libcublas.so.12" in syms
    assert all(s.split("@@")[0].startswith(("cublas", "vkzb", "libcublas")) for s in syms), "only cublas* and vkzb* are exported"
    lt = _dynamic_symbols("libcublasLt.so.12")
    assert "cublasLtMatmul@@libcublasLt.so.12" in lt
    assert not any(s.startswith("cublasGemmEx") for s in lt)
    soname = subprocess.run(["readelf", "-d", str(vk.LIB_DIR / "libcublas.so.12")], capture_output=True, text=True).stdout
    assert "libcublas.so.12" in soname and "libcublasLt" not in soname


def test_stub_surface_answers_not_supported():
    lib = vk.cublas_library()
    names = (ROOT / "vulkanizer_b200" / "csrc" / "blas_stub_names.def").read_text().split()
    assert len(names) >= 227
    for name in names[:5] + ["cublasStrsv_v2", "cublasZgemm_v2"]:
        fn = getattr(lib, name)
        fn.restype = C.c_int
        assert fn() == capi.STATUS_NOT_SUPPORTED
    # the triangular solves and batched factorizations are served, not stubs: a null handle says so
    assert "cublasStrsm_v2" not in names and "cublasSgetrfBatched" not in names
    assert lib.cublasStrsm_v2(None, 0, 0, 0, 0, 1, 1, None, None, 1, None, 1) == capi.STATUS_NOT_INITIALIZED
    assert lib.cublasSgeqrfBatched(None, 1, 1, None, 1, None, None, 1) == capi.STATUS_NOT_INITIALIZED


def test_null_handle_and_status_strings():
    lib = vk.cublas_library()
    assert lib.cublasSgemm_v2(None, 0, 0, 1, 1, 1, None, None, 1, None, 1, None, None, 1) == capi.STATUS_NOT_INITIALIZED
    assert lib.cublasSetStream_v2(None, None) == capi.STATUS_NOT_INITIALIZED
    assert lib.cublasDestroy_v2(None) == capi.STATUS_NOT_INITIALIZED
    assert lib.cublasCreate_v2(None) == capi.STATUS_INVALID_VALUE
    assert lib.cublasGetStatusName(15) == b"CUBLAS_STATUS_NOT_SUPPORTED"
    assert lib.cublasGetStatusString(0) == b"success"
    assert lib.cublasGetStatusName(1234) == b"CUBLAS_STATUS_UNKNOWN"
    v = C.c_int(0)
    assert lib.cublasGetVersion_v2(None, C.byref(v)) == 0 and v.value == 120900
    assert lib.cublasSgemv_v2(None, 0, 1, 1, None, None, 1, None, 1, None, None, 1) == capi.STATUS_NOT_INITIALIZED
    assert lib.cublasSgemm_v2_64(None, 0, 0, 1 << 33, 1, 1, None, None, 1, None, 1, None, None, 1) == capi.STATUS_NOT_SUPPORTED


def test_lt_descriptor_plumbing():
    lib = vk.cublaslt_library()
    desc = C.c_void_p()
    assert lib.cublasLtMatmulDescCreate(C.byref(desc), capi.COMPUTE_32F, capi.CUDA_R_32F) == 0
    val = C.c_int32(capi.OP_T)
    assert lib.cublasLtMatmulDescSetAttribute(desc, capi.LT_DESC_TRANSA, C.addressof(val), 4) == 0
    out, written = C.c_int32(-1), C.c_size_t(0)
    assert lib.cublasLtMatmulDescGetAttribute(desc, capi.LT_DESC_TRANSA, C.addressof(out), 4, C.byref(written)) == 0
    assert out.value == capi.OP_T and written.value == 4
    assert lib.cublasLtMatmulDescSetAttribute(desc, capi.LT_DESC_TRANSA, C.addressof(val), 2) == capi.STATUS_INVALID_VALUE  # wrong size
    assert lib.cublasLtMatmulDescSetAttribute(desc, 11, C.addressof(val), 4) == capi.STATUS_INVALID_VALUE  # aux pointer: 8 bytes
    ptr = C.c_void_p(0x1000)
    assert lib.cublasLtMatmulDescSetAttribute(desc, capi.LT_DESC_AUX_POINTER, C.addressof(ptr), 8) == 0
    back = C.c_void_p(0)
    assert lib.cublasLtMatmulDescGetAttribute(desc, capi.LT_DESC_AUX_POINTER, C.addressof(back), 8, None) == 0 and back.value == 0x1000
    assert lib.cublasLtMatmulDescSetAttribute(desc, 17, C.addressof(val), 8) == capi.STATUS_NOT_SUPPORTED  # A scale pointer (fp8): not served
    assert lib.cublasLtMatmulDescSetAttribute(desc, 15, C.addressof(val), 4) == 0  # SM count target: accepted hint
    # size query with a null buffer
    assert lib.cublasLtMatmulDescGetAttribute(desc, capi.LT_DESC_EPILOGUE, None, 0, C.byref(written)) == 0 and written.value == 4
    layout = C.c_void_p()
    assert lib.cublasLtMatrixLayoutCreate(C.byref(layout), capi.CUDA_R_16F, 64, 32, 64) == 0
    ld, n64 = C.c_int64(0), C.c_uint64(0)
    assert lib.cublasLtMatrixLayoutGetAttribute(layout, capi.LT_LAYOUT_LD, C.addressof(ld), 8, None) == 0 and ld.value == 64
    assert lib.cublasLtMatrixLayoutGetAttribute(layout, capi.LT_LAYOUT_ROWS, C.addressof(n64), 8, None) == 0 and n64.value == 64
    pref = C.c_void_p()
    assert lib.cublasLtMatmulPreferenceCreate(C.byref(pref)) == 0
    ws = C.c_uint64(1 << 20)
    assert lib.cublasLtMatmulPreferenceSetAttribute(pref, capi.LT_PREF_MAX_WORKSPACE_BYTES, C.addressof(ws), 8) == 0
    # a missing handle is an invalid value for the heuristic and NOT_INITIALIZED for the matmul
    heur, found = C.create_string_buffer(96), C.c_int(7)
    assert lib.cublasLtMatmulAlgoGetHeuristic(None, desc, layout, layout, layout, layout, pref, 1, C.addressof(heur), C.byref(found)) == capi.STATUS_INVALID_VALUE
    assert lib.cublasLtMatmul(None, desc, None, None, layout, None, layout, None, None, layout, None, layout, None, None, 0, None) == capi.STATUS_NOT_INITIALIZED
    assert lib.cublasLtMatmulPreferenceDestroy(pref) == 0 and lib.cublasLtMatrixLayoutDestroy(layout) == 0 and lib.cublasLtMatmulDescDestroy(desc) == 0


def _enum_values(text):
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    return {m.group(1): int(m.group(2), 0) for m in re.finditer(r"\b((?:CUBLASLT|CUBLAS|CUDA_[RC])_[A-Z0-9_]+)\s*=\s*(-?(?:0x[0-9a-fA-F]+|\d+))\s*[,}]", text)}


@pytest.mark.parametrize("mine, theirs", [("vkzb_cublas.h", ["cublas_api.h", "library_types.h"]), ("vkzb_cublaslt.h", ["cublasLt.h"])])
def test_enum_values_agree_with_the_cuda_toolkit(mine, theirs):
    toolkit = Path("/usr/local/cuda/include")
    if not all((toolkit / t).exists() for t in theirs):
        pytest.skip("CUDA toolkit headers not present")
    ours = _enum_values((ROOT / "include" / mine).read_text())
    nvidia = {}
    for t in theirs:
        nvidia.update(_enum_values((toolkit / t).read_text()))
    shared = sorted(set(ours) & set(nvidia))
    assert len(shared) >= 20, shared
    assert {k: ours[k] for k in shared} == {k: nvidia[k] for k in shared}
