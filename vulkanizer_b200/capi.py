"""ctypes binding to the C ABI of libcublas.so.12 and libcublasLt.so.12 built from ``csrc/``.

Enum values are those of ``include/vkzb_cublas.h`` / ``include/vkzb_cublaslt.h`` (NVIDIA's documented ones).
Pointers are passed as integers (``tensor.data_ptr()``); scalars alpha/beta are packed on the host in the
scalar type the compute type calls for, as the C callers of k0zi/Vulkanizer's tests do (tests/cublas.cpp:138-144).
"""
from __future__ import annotations

import ctypes as C
import os
import re
import struct
import subprocess
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
# VKZB_LIB_DIR: load the libraries from another build directory (e.g. lib_measure, made by `make MEASURE=1`)
LIB_DIR = Path(os.environ["VKZB_LIB_DIR"]).resolve() if os.environ.get("VKZB_LIB_DIR") else PKG_DIR / "lib"
INCLUDE_DIR = PKG_DIR.parent / "include"

# ---- enum values (include/vkzb_cublas.h) ----
CUDA_R_32F, CUDA_R_64F, CUDA_R_16F, CUDA_R_8I, CUDA_R_32I, CUDA_R_16BF = 0, 1, 2, 3, 10, 14
OP_N, OP_T, OP_C = 0, 1, 2
FILL_LOWER, FILL_UPPER, DIAG_NON_UNIT, DIAG_UNIT, SIDE_LEFT, SIDE_RIGHT = 0, 1, 0, 1, 0, 1
POINTER_MODE_HOST, POINTER_MODE_DEVICE = 0, 1
DEFAULT_MATH, TF32_TENSOR_OP_MATH = 0, 3
COMPUTE_16F, COMPUTE_32F, COMPUTE_64F, COMPUTE_32I = 64, 68, 70, 72
COMPUTE_32F_FAST_16F, COMPUTE_32F_FAST_TF32 = 74, 77
GEMM_DEFAULT, GEMM_DEFAULT_TENSOR_OP = -1, 99
STATUS = {0: "SUCCESS", 1: "NOT_INITIALIZED", 3: "ALLOC_FAILED", 7: "INVALID_VALUE", 8: "ARCH_MISMATCH",
          11: "MAPPING_ERROR", 13: "EXECUTION_FAILED", 14: "INTERNAL_ERROR", 15: "NOT_SUPPORTED", 16: "LICENSE_ERROR"}
STATUS_SUCCESS, STATUS_NOT_INITIALIZED, STATUS_INVALID_VALUE, STATUS_NOT_SUPPORTED = 0, 1, 7, 15
# kernel families (include/vkzb_ext.h)
PATH_NONE, PATH_SCALE, PATH_GENERIC, PATH_GEMV, PATH_SGEMM, PATH_UMMA, PATH_DGEMM = range(7)
# cuBLASLt (include/vkzb_cublaslt.h)
LT_EPILOGUE_DEFAULT, LT_EPILOGUE_RELU, LT_EPILOGUE_BIAS, LT_EPILOGUE_RELU_BIAS = 1, 2, 4, 6
LT_EPILOGUE_GELU, LT_EPILOGUE_GELU_BIAS = 32, 36
LT_EPILOGUE_RELU_AUX, LT_EPILOGUE_RELU_AUX_BIAS, LT_EPILOGUE_GELU_AUX, LT_EPILOGUE_GELU_AUX_BIAS = 130, 134, 160, 164
LT_EPILOGUE_DRELU, LT_EPILOGUE_DRELU_BGRAD, LT_EPILOGUE_DGELU, LT_EPILOGUE_DGELU_BGRAD = 136, 152, 192, 208
LT_EPILOGUE_BGRADA, LT_EPILOGUE_BGRADB = 256, 512
LT_DESC_AUX_POINTER, LT_DESC_AUX_LD, LT_DESC_AUX_BATCH_STRIDE, LT_DESC_AUX_DATA_TYPE = 11, 12, 13, 22
LT_ORDER_COL, LT_ORDER_ROW = 0, 1
LT_DESC_COMPUTE_TYPE, LT_DESC_SCALE_TYPE, LT_DESC_POINTER_MODE, LT_DESC_TRANSA, LT_DESC_TRANSB, LT_DESC_TRANSC = range(6)
LT_DESC_EPILOGUE, LT_DESC_BIAS_POINTER, LT_DESC_BIAS_BATCH_STRIDE, LT_DESC_BIAS_DATA_TYPE = 7, 8, 10, 26
LT_LAYOUT_TYPE, LT_LAYOUT_ORDER, LT_LAYOUT_ROWS, LT_LAYOUT_COLS, LT_LAYOUT_LD, LT_LAYOUT_BATCH_COUNT, LT_LAYOUT_BATCH_STRIDE = range(7)
LT_PREF_MAX_WORKSPACE_BYTES = 1


class BlasError(RuntimeError):
    def __init__(self, call: str, status: int):
        super().__init__(f"{call} returned CUBLAS_STATUS_{STATUS.get(status, status)}")
        self.status = status


def build_libraries(jobs: int = 8) -> None:
    """Compiles csrc/ for sm_100a into lib/ (nvcc cross-compiles without a GPU)."""
    subprocess.run(["make", "-C", str(PKG_DIR / "csrc"), f"-j{jobs}", "all"], check=True)


def _load(name: str) -> C.CDLL:
    path = LIB_DIR / name
    if not path.exists():
        raise RuntimeError(f"{path} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                           f"(there is no fallback implementation)")
    # by absolute path and RTLD_LOCAL: another libcublas.so.12 already in the process (PyTorch's) is left alone
    return C.CDLL(str(path), mode=os.RTLD_LOCAL | os.RTLD_NOW)


_cublas = None
_cublaslt = None
_vp, _i, _ll, _sz = C.c_void_p, C.c_int, C.c_longlong, C.c_size_t


class AttentionProblem(C.Structure):
    """vkzbAttentionProblem of include/vkzb_attention.h."""
    _fields_ = ([(n, _i) for n in ("dataType", "batches", "heads", "kvHeads", "numQ", "numK", "headDim", "mask")] + [("scale", C.c_float)] +
                [f for t in "qkvo" for f in ((t, _vp), (t + "Row", _ll), (t + "Head", _ll), (t + "Batch", _ll))] + [("logSumExp", _vp)])


def cublas_library() -> C.CDLL:
    global _cublas
    if _cublas is None:
        lib = _load("libcublas.so.12")
        gemm_head = [_vp, _i, _i, _i, _i, _i]  # handle, transa, transb, m, n, k
        protos = {
            "cublasCreate_v2": [C.POINTER(_vp)],
            "cublasDestroy_v2": [_vp],
            "cublasGetVersion_v2": [_vp, C.POINTER(_i)],
            "cublasSetStream_v2": [_vp, _vp],
            "cublasGetStream_v2": [_vp, C.POINTER(_vp)],
            "cublasSetWorkspace_v2": [_vp, _vp, _sz],
            "cublasSetPointerMode_v2": [_vp, _i],
            "cublasGetPointerMode_v2": [_vp, C.POINTER(_i)],
            "cublasSetMathMode": [_vp, _i],
            "cublasGetMathMode": [_vp, C.POINTER(_i)],
            "cublasSetAtomicsMode": [_vp, _i],
            "cublasGetAtomicsMode": [_vp, C.POINTER(_i)],
            "cublasSetSmCountTarget": [_vp, _i],
            "cublasSgemm_v2": gemm_head + [_vp, _vp, _i, _vp, _i, _vp, _vp, _i],
            "cublasDgemm_v2": gemm_head + [_vp, _vp, _i, _vp, _i, _vp, _vp, _i],
            "cublasSgemm_v2_64": [_vp, _i, _i, _ll, _ll, _ll, _vp, _vp, _ll, _vp, _ll, _vp, _vp, _ll],
            "cublasSgemmStridedBatched": gemm_head + [_vp, _vp, _i, _ll, _vp, _i, _ll, _vp, _vp, _i, _ll, _i],
            "cublasDgemmStridedBatched": gemm_head + [_vp, _vp, _i, _ll, _vp, _i, _ll, _vp, _vp, _i, _ll, _i],
            "cublasSgemmBatched": gemm_head + [_vp, _vp, _i, _vp, _i, _vp, _vp, _i, _i],
            "cublasGemmEx": gemm_head + [_vp, _vp, _i, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i],
            "cublasHgemm": gemm_head + [_vp, _vp, _i, _vp, _i, _vp, _vp, _i],
            "cublasSgemmEx": gemm_head + [_vp, _vp, _i, _i, _vp, _i, _i, _vp, _vp, _i, _i],
            "cublasGemmBatchedEx": gemm_head + [_vp, _vp, _i, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i],
            "cublasGemmStridedBatchedEx": gemm_head + [_vp, _vp, _i, _i, _ll, _vp, _i, _i, _ll, _vp, _vp, _i, _i, _ll, _i, _i, _i],
            "cublasGemmGroupedBatchedEx": [_vp] + [_vp] * 6 + [_vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _vp, _i, _vp, _i],
            "cublasSgemv_v2": [_vp, _i, _i, _i, _vp, _vp, _i, _vp, _i, _vp, _vp, _i],
            "cublasSgemv_v2_64": [_vp, _i, _ll, _ll, _vp, _vp, _ll, _vp, _ll, _vp, _vp, _ll],
            # handle, side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb (, batch)
            "cublasStrsm_v2": [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _vp, _i],
            "cublasDtrsm_v2": [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _vp, _i],
            "cublasStrsmBatched": [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _vp, _i, _i],
            "cublasDtrsmBatched": [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _vp, _i, _i],
            "cublasSgetrfBatched": [_vp, _i, _vp, _i, _vp, _vp, _i],
            "cublasDgetrfBatched": [_vp, _i, _vp, _i, _vp, _vp, _i],
            "cublasSgetrsBatched": [_vp, _i, _i, _i, _vp, _i, _vp, _vp, _i, C.POINTER(_i), _i],
            "cublasDgetrsBatched": [_vp, _i, _i, _i, _vp, _i, _vp, _vp, _i, C.POINTER(_i), _i],
            "cublasSgeqrfBatched": [_vp, _i, _i, _vp, _i, _vp, C.POINTER(_i), _i],
            "cublasDgeqrfBatched": [_vp, _i, _i, _vp, _i, _vp, C.POINTER(_i), _i],
        }
        for name, args in protos.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, _i
        lib.cublasGetStatusName.argtypes, lib.cublasGetStatusName.restype = [_i], C.c_char_p
        lib.cublasGetStatusString.argtypes, lib.cublasGetStatusString.restype = [_i], C.c_char_p
        lib.cublasGetCudartVersion.argtypes, lib.cublasGetCudartVersion.restype = [], _sz
        lib.vkzbLaunchCount.argtypes, lib.vkzbLaunchCount.restype = [], C.c_uint64
        lib.vkzbLastPath.argtypes, lib.vkzbLastPath.restype = [], _i
        lib.vkzbLastPlan.argtypes, lib.vkzbLastPlan.restype = [], _i
        lib.vkzbDeviceStatus.argtypes, lib.vkzbDeviceStatus.restype = [], _i
        lib.vkzbSetOutputMirrors.argtypes, lib.vkzbSetOutputMirrors.restype = [_vp, _vp, _sz, _i, C.POINTER(_vp)], _i
        lib.vkzbSgemmStaticScratch.argtypes = [_vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _vp, _i, _vp, _vp, _i]
        lib.vkzbSgemmStaticScratch.restype = _i
        lib.vkzbAttentionForward.argtypes, lib.vkzbAttentionForward.restype = [_vp, C.POINTER(AttentionProblem)], _i
        lib.vkzbAttentionStatus.argtypes, lib.vkzbAttentionStatus.restype = [], _i
        _cublas = lib
    return _cublas


def attention_forward(stream, data_type, batches, heads, kv_heads, num_q, num_k, head_dim, mask, scale, q, q_strides, k, k_strides, v, v_strides,
                      o, o_strides, log_sum_exp=None) -> int:
    """vkzbAttentionForward (include/vkzb_attention.h): O = softmax(scale Q K^T + mask) V on device pointers. Each *_strides is
    (row, head, batch) in elements. Returns the status; raises nothing, so tests can check refusals."""
    a = AttentionProblem(data_type, batches, heads, kv_heads, num_q, num_k, head_dim, mask, scale, q, *q_strides, k, *k_strides, v, *v_strides,
                         o, *o_strides, log_sum_exp)
    return cublas_library().vkzbAttentionForward(stream, C.byref(a))


def cublaslt_library() -> C.CDLL:
    global _cublaslt
    if _cublaslt is None:
        lib = _load("libcublasLt.so.12")
        protos = {
            "cublasLtCreate": [C.POINTER(_vp)],
            "cublasLtDestroy": [_vp],
            "cublasLtMatmulDescCreate": [C.POINTER(_vp), _i, _i],
            "cublasLtMatmulDescDestroy": [_vp],
            "cublasLtMatmulDescSetAttribute": [_vp, _i, _vp, _sz],
            "cublasLtMatmulDescGetAttribute": [_vp, _i, _vp, _sz, C.POINTER(_sz)],
            "cublasLtMatrixLayoutCreate": [C.POINTER(_vp), _i, C.c_uint64, C.c_uint64, C.c_int64],
            "cublasLtMatrixLayoutDestroy": [_vp],
            "cublasLtMatrixLayoutSetAttribute": [_vp, _i, _vp, _sz],
            "cublasLtMatrixLayoutGetAttribute": [_vp, _i, _vp, _sz, C.POINTER(_sz)],
            "cublasLtMatmulPreferenceCreate": [C.POINTER(_vp)],
            "cublasLtMatmulPreferenceDestroy": [_vp],
            "cublasLtMatmulPreferenceSetAttribute": [_vp, _i, _vp, _sz],
            "cublasLtMatmulAlgoGetHeuristic": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, C.POINTER(_i)],
            "cublasLtMatmul": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp],
        }
        for name, args in protos.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, _i
        lib.cublasLtGetVersion.argtypes, lib.cublasLtGetVersion.restype = [], _sz
        lib.vkzbLaunchCount.argtypes, lib.vkzbLaunchCount.restype = [], C.c_uint64
        lib.vkzbLastPath.argtypes, lib.vkzbLastPath.restype = [], _i
        lib.vkzbDeviceStatus.argtypes, lib.vkzbDeviceStatus.restype = [], _i
        lib.vkzbSetOutputMirrors.argtypes, lib.vkzbSetOutputMirrors.restype = [_vp, _vp, _sz, _i, C.POINTER(_vp)], _i
        _cublaslt = lib
    return _cublaslt


_nccl = None
NCCL_TYPES = {"int8": 0, "uint8": 1, "int32": 2, "uint32": 3, "int64": 4, "uint64": 5, "float16": 6, "float32": 7, "float64": 8, "bfloat16": 9}
NCCL_SUM, NCCL_PROD, NCCL_MAX, NCCL_MIN, NCCL_AVG = range(5)


class NcclUniqueId(C.Structure):
    _fields_ = [("internal", C.c_char * 128)]


def nccl_library() -> C.CDLL:
    global _nccl
    if _nccl is None:
        lib = _load("libnccl.so.2")
        coll = [_vp, _vp, _sz, _i]
        protos = {
            "ncclGetVersion": [C.POINTER(_i)],
            "ncclGetUniqueId": [C.POINTER(NcclUniqueId)],
            "ncclCommInitRank": [C.POINTER(_vp), _i, NcclUniqueId, _i],
            "ncclCommInitAll": [C.POINTER(_vp), _i, C.POINTER(_i)],
            "ncclCommDestroy": [_vp],
            "ncclCommAbort": [_vp],
            "ncclCommCount": [_vp, C.POINTER(_i)],
            "ncclCommUserRank": [_vp, C.POINTER(_i)],
            "ncclCommCuDevice": [_vp, C.POINTER(_i)],
            "ncclCommGetAsyncError": [_vp, C.POINTER(_i)],
            "ncclAllGather": coll + [_vp, _vp],
            "ncclAllReduce": coll + [_i, _vp, _vp],
            "ncclReduceScatter": coll + [_i, _vp, _vp],
            "ncclReduce": coll + [_i, _i, _vp, _vp],
            "ncclBroadcast": coll + [_i, _vp, _vp],
            "ncclGather": coll + [_i, _vp, _vp],
            "ncclAlltoAll": coll + [_vp, _vp],
            "ncclGroupStart": [],
            "ncclGroupEnd": [],
            "ncclSend": [_vp, _sz, _i, _i, _vp, _vp],
            "ncclRecv": [_vp, _sz, _i, _i, _vp, _vp],
            "ncclCommSplit": [_vp, _i, _i, C.POINTER(_vp), _vp],
            "ncclRedOpCreatePreMulSum": [C.POINTER(_i), _vp, _i, _i, _vp],
            "ncclRedOpDestroy": [_i, _vp],
            "vkzbNcclSelfTestLostPeer": [_vp, _vp],
            "vkzbNcclExchangeBuffer": [_vp, _vp, C.POINTER(_vp)],
            "vkzbNcclBarrier": [_vp, _vp],
        }
        for name, args in protos.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, _i
        lib.ncclGetErrorString.argtypes, lib.ncclGetErrorString.restype = [_i], C.c_char_p
        lib.ncclGetLastError.argtypes, lib.ncclGetLastError.restype = [_vp], C.c_char_p
        _nccl = lib
    return _nccl


class NcclError(RuntimeError):
    pass


class NcclComm:
    """One communicator of this repository's libnccl.so.2. The 128-byte unique id travels between the ranks by any means the
    caller has (the benchmark broadcasts it with torch.distributed, as an MPI program would with MPI_Bcast)."""

    def __init__(self, nranks: int, rank: int, unique_id: bytes, _adopt=None):
        self.lib = nccl_library()
        if _adopt is not None:  # a communicator made by ncclCommSplit
            self.comm, self.nranks, self.rank = _adopt, nranks, rank
            return
        uid = NcclUniqueId()
        C.memmove(C.addressof(uid), unique_id, 128)
        comm = _vp()
        self._check("ncclCommInitRank", self.lib.ncclCommInitRank(C.byref(comm), nranks, uid, rank), None)
        self.comm, self.nranks, self.rank = comm, nranks, rank

    @staticmethod
    def unique_id() -> bytes:
        uid = NcclUniqueId()
        status = nccl_library().ncclGetUniqueId(C.byref(uid))
        if status:
            raise NcclError(f"ncclGetUniqueId: {status}")
        return C.string_at(C.addressof(uid), 128)

    def _check(self, call, status, comm):
        if status:
            detail = self.lib.ncclGetLastError(comm).decode() if comm else ""
            raise NcclError(f"{call}: {self.lib.ncclGetErrorString(status).decode()} ({detail})")

    def all_gather(self, send, recv, count, dtype, stream=0):
        self._check("ncclAllGather", self.lib.ncclAllGather(send, recv, count, NCCL_TYPES[dtype], self.comm, stream), self.comm)

    def all_reduce(self, send, recv, count, dtype, op=NCCL_SUM, stream=0):
        self._check("ncclAllReduce", self.lib.ncclAllReduce(send, recv, count, NCCL_TYPES[dtype], op, self.comm, stream), self.comm)

    def reduce_scatter(self, send, recv, recvcount, dtype, op=NCCL_SUM, stream=0):
        self._check("ncclReduceScatter", self.lib.ncclReduceScatter(send, recv, recvcount, NCCL_TYPES[dtype], op, self.comm, stream), self.comm)

    def reduce(self, send, recv, count, dtype, root, op=NCCL_SUM, stream=0):
        self._check("ncclReduce", self.lib.ncclReduce(send, recv, count, NCCL_TYPES[dtype], op, root, self.comm, stream), self.comm)

    def broadcast(self, send, recv, count, dtype, root, stream=0):
        self._check("ncclBroadcast", self.lib.ncclBroadcast(send, recv, count, NCCL_TYPES[dtype], root, self.comm, stream), self.comm)

    def gather(self, send, recv, count, dtype, root, stream=0):
        self._check("ncclGather", self.lib.ncclGather(send, recv, count, NCCL_TYPES[dtype], root, self.comm, stream), self.comm)

    def all_to_all(self, send, recv, count, dtype, stream=0):
        self._check("ncclAlltoAll", self.lib.ncclAlltoAll(send, recv, count, NCCL_TYPES[dtype], self.comm, stream), self.comm)

    def send(self, buf, count, dtype, peer, stream=0):
        self._check("ncclSend", self.lib.ncclSend(buf, count, NCCL_TYPES[dtype], peer, self.comm, stream), self.comm)

    def recv(self, buf, count, dtype, peer, stream=0):
        self._check("ncclRecv", self.lib.ncclRecv(buf, count, NCCL_TYPES[dtype], peer, self.comm, stream), self.comm)

    def group_start(self):
        self._check("ncclGroupStart", self.lib.ncclGroupStart(), None)

    def group_end(self):
        self._check("ncclGroupEnd", self.lib.ncclGroupEnd(), self.comm)

    def split(self, color: int, key: int):
        """The communicator of the ranks that passed `color` (None for NCCL_SPLIT_NOCOLOR = -1)."""
        new = _vp()
        self._check("ncclCommSplit", self.lib.ncclCommSplit(self.comm, color, key, C.byref(new), None), self.comm)
        if not new.value:
            return None
        count, rank = _i(0), _i(0)
        self.lib.ncclCommCount(new, C.byref(count))
        self.lib.ncclCommUserRank(new, C.byref(rank))
        return NcclComm(count.value, rank.value, b"", _adopt=new)

    def premul_sum(self, factor: float) -> int:
        """A reduction operator that multiplies this rank's contribution by `factor` (a host float) before the sum."""
        op, value = _i(0), C.c_float(factor)
        self._check("ncclRedOpCreatePreMulSum", self.lib.ncclRedOpCreatePreMulSum(C.byref(op), C.addressof(value), NCCL_TYPES["float32"], 1, self.comm), self.comm)
        return op.value

    def destroy_op(self, op: int):
        self._check("ncclRedOpDestroy", self.lib.ncclRedOpDestroy(op, self.comm), self.comm)

    def self_test_lost_peer(self, stream=0):
        self._check("vkzbNcclSelfTestLostPeer", self.lib.vkzbNcclSelfTestLostPeer(self.comm, stream), self.comm)

    def abort(self):
        self.lib.ncclCommAbort(self.comm)

    def exchange_buffer(self, ptr: int) -> list[int]:
        """Addresses through which this process reaches each rank's buffer (extension vkzbNcclExchangeBuffer)."""
        out = (_vp * self.nranks)()
        self._check("vkzbNcclExchangeBuffer", self.lib.vkzbNcclExchangeBuffer(self.comm, ptr, out), self.comm)
        return [int(out[i] or 0) for i in range(self.nranks)]

    def barrier(self, stream=0):
        self._check("vkzbNcclBarrier", self.lib.vkzbNcclBarrier(self.comm, stream), self.comm)

    def async_error(self) -> int:
        out = _i(0)
        self.lib.ncclCommGetAsyncError(self.comm, C.byref(out))
        return out.value

    def destroy(self):
        if self.comm is not None:
            self.lib.ncclCommDestroy(self.comm)
            self.comm = None


def declared_symbols(header: str) -> list[str]:
    """Function names a header under include/ declares (for the export check)."""
    text = (INCLUDE_DIR / header).read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:cublas|cublasLt|nccl|vkzb)[A-Za-z0-9_]*)\s*\(", text)))


def pack_scalar(value, compute_type: int) -> bytes:
    """alpha / beta in the scalar type of the compute type: half, int32, double, else float."""
    if compute_type in (64, 65):
        import numpy as np
        return np.float16(value).tobytes()
    if compute_type in (72, 73):
        return struct.pack("<i", int(value))
    if compute_type in (70, 71):
        return struct.pack("<d", float(value))
    return struct.pack("<f", float(value))


class Cublas:
    """One cuBLAS handle. Methods take raw device addresses and return nothing; a non-zero status raises BlasError
    unless ``check=False``, in which case the status is returned."""

    def __init__(self):
        self.lib = cublas_library()
        h = _vp()
        status = self.lib.cublasCreate_v2(C.byref(h))
        if status:
            raise BlasError("cublasCreate_v2", status)
        self.handle = h
        self._keep = []

    def destroy(self):
        if self.handle is not None:
            self.lib.cublasDestroy_v2(self.handle)
            self.handle = None

    def _done(self, call, status, check):
        if check and status:
            raise BlasError(call, status)
        return status

    def set_stream(self, stream: int):
        return self._done("cublasSetStream_v2", self.lib.cublasSetStream_v2(self.handle, stream), True)

    def set_pointer_mode(self, mode: int):
        return self._done("cublasSetPointerMode_v2", self.lib.cublasSetPointerMode_v2(self.handle, mode), True)

    def set_math_mode(self, mode: int):
        return self._done("cublasSetMathMode", self.lib.cublasSetMathMode(self.handle, mode), True)

    def _scalars(self, alpha, beta, compute, device_scalars):
        if device_scalars:  # already device addresses
            return alpha, beta
        a = C.create_string_buffer(pack_scalar(alpha, compute), 8)
        b = C.create_string_buffer(pack_scalar(beta, compute), 8)
        self._keep = [a, b]
        return C.addressof(a), C.addressof(b)

    def sgemm(self, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, Cp, ldc, check=True, device_scalars=False):
        a, b = self._scalars(alpha, beta, COMPUTE_32F, device_scalars)
        return self._done("cublasSgemm_v2", self.lib.cublasSgemm_v2(self.handle, ta, tb, m, n, k, a, A, lda, B, ldb, b, Cp, ldc), check)

    def dgemm(self, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, Cp, ldc, check=True):
        a, b = self._scalars(alpha, beta, COMPUTE_64F, False)
        return self._done("cublasDgemm_v2", self.lib.cublasDgemm_v2(self.handle, ta, tb, m, n, k, a, A, lda, B, ldb, b, Cp, ldc), check)

    def gemm_ex(self, ta, tb, m, n, k, alpha, A, type_a, lda, B, type_b, ldb, beta, Cp, type_c, ldc, compute=COMPUTE_32F,
                algo=GEMM_DEFAULT, check=True, device_scalars=False):
        a, b = self._scalars(alpha, beta, compute, device_scalars)
        return self._done("cublasGemmEx", self.lib.cublasGemmEx(self.handle, ta, tb, m, n, k, a, A, type_a, lda, B, type_b, ldb, b,
                                                                Cp, type_c, ldc, compute, algo), check)

    def gemm_strided_batched_ex(self, ta, tb, m, n, k, alpha, A, type_a, lda, stride_a, B, type_b, ldb, stride_b, beta, Cp,
                                type_c, ldc, stride_c, batch, compute=COMPUTE_32F, algo=GEMM_DEFAULT, check=True,
                                device_scalars=False):
        a, b = self._scalars(alpha, beta, compute, device_scalars)
        return self._done("cublasGemmStridedBatchedEx",
                          self.lib.cublasGemmStridedBatchedEx(self.handle, ta, tb, m, n, k, a, A, type_a, lda, stride_a, B, type_b,
                                                              ldb, stride_b, b, Cp, type_c, ldc, stride_c, batch, compute, algo), check)

    def gemm_batched_ex(self, ta, tb, m, n, k, alpha, A_array, type_a, lda, B_array, type_b, ldb, beta, C_array, type_c, ldc,
                        batch, compute=COMPUTE_32F, algo=GEMM_DEFAULT, check=True):
        a, b = self._scalars(alpha, beta, compute, False)
        return self._done("cublasGemmBatchedEx",
                          self.lib.cublasGemmBatchedEx(self.handle, ta, tb, m, n, k, a, A_array, type_a, lda, B_array, type_b, ldb, b,
                                                       C_array, type_c, ldc, batch, compute, algo), check)

    def sgemv(self, trans, m, n, alpha, A, lda, x, incx, beta, y, incy, check=True):
        a, b = self._scalars(alpha, beta, COMPUTE_32F, False)
        return self._done("cublasSgemv_v2", self.lib.cublasSgemv_v2(self.handle, trans, m, n, a, A, lda, x, incx, b, y, incy), check)

    def last_path(self) -> int:
        return self.lib.vkzbLastPath()

    def last_plan(self) -> dict:
        """Layout of this thread's most recent tensor-core launch (extension vkzbLastPlan)."""
        bits = self.lib.vkzbLastPlan()
        return {"bn": bits & 1023, "pair": bool(bits >> 10 & 1), "wide": bool(bits >> 11 & 1), "splits": bits >> 12 & 15}

    def launch_count(self) -> int:
        return self.lib.vkzbLaunchCount()

    def set_output_mirrors(self, local_base: int, nbytes: int, mirrors: list[int]):
        """Every later GEMM on this handle whose result lies in [local_base, local_base + nbytes) also writes it, tile by
        tile, to the same offset in the `mirrors` buffers (extension vkzbSetOutputMirrors); an empty list switches it off."""
        arr = (_vp * max(1, len(mirrors)))(*mirrors)
        status = self.lib.vkzbSetOutputMirrors(self.handle, local_base, nbytes, len(mirrors), arr)
        if status:
            raise BlasError("vkzbSetOutputMirrors", status)

    def device_status(self) -> int:
        return self.lib.vkzbDeviceStatus()


class CublasLt:
    """cuBLASLt handle plus a helper that builds the descriptors for one matmul, runs it and frees them."""

    def __init__(self):
        self.lib = cublaslt_library()
        h = _vp()
        status = self.lib.cublasLtCreate(C.byref(h))
        if status:
            raise BlasError("cublasLtCreate", status)
        self.handle = h

    def destroy(self):
        if self.handle is not None:
            self.lib.cublasLtDestroy(self.handle)
            self.handle = None

    def _set(self, fn, obj, attr, ctype, value):
        v = ctype(value)
        status = fn(obj, attr, C.addressof(v), C.sizeof(v))
        if status:
            raise BlasError(fn.__name__, status)

    def matmul(self, ta, tb, m, n, k, alpha, A, type_a, lda, B, type_b, ldb, beta, Cp, type_c, ldc, D, type_d, ldd, *,
               compute=COMPUTE_32F, scale_type=CUDA_R_32F, epilogue=LT_EPILOGUE_DEFAULT, bias=0, bias_type=None, batch=1,
               stride_a=0, stride_b=0, stride_c=0, stride_d=0, stream=0, check=True, order=None, aux=0, aux_ld=0, aux_stride=0,
               aux_type=None):
        """One cublasLtMatmul. `order` is None (column order), one LT_ORDER_* for all four matrices, or a tuple (A, B, C, D)."""
        lib = self.lib
        desc = _vp()
        status = lib.cublasLtMatmulDescCreate(C.byref(desc), compute, scale_type)
        if status:
            raise BlasError("cublasLtMatmulDescCreate", status)
        layouts = []
        try:
            self._set(lib.cublasLtMatmulDescSetAttribute, desc, LT_DESC_TRANSA, C.c_int32, ta)
            self._set(lib.cublasLtMatmulDescSetAttribute, desc, LT_DESC_TRANSB, C.c_int32, tb)
            self._set(lib.cublasLtMatmulDescSetAttribute, desc, LT_DESC_EPILOGUE, C.c_uint32, epilogue)
            if bias:
                self._set(lib.cublasLtMatmulDescSetAttribute, desc, LT_DESC_BIAS_POINTER, C.c_void_p, bias)
            if bias_type is not None:
                self._set(lib.cublasLtMatmulDescSetAttribute, desc, LT_DESC_BIAS_DATA_TYPE, C.c_int32, bias_type)
            if aux:
                self._set(lib.cublasLtMatmulDescSetAttribute, desc, LT_DESC_AUX_POINTER, C.c_void_p, aux)
                self._set(lib.cublasLtMatmulDescSetAttribute, desc, LT_DESC_AUX_LD, C.c_int64, aux_ld)
                self._set(lib.cublasLtMatmulDescSetAttribute, desc, LT_DESC_AUX_BATCH_STRIDE, C.c_int64, aux_stride)
            if aux_type is not None:
                self._set(lib.cublasLtMatmulDescSetAttribute, desc, LT_DESC_AUX_DATA_TYPE, C.c_int32, aux_type)
            orders = (order,) * 4 if order is None or isinstance(order, int) else tuple(order)
            rows_a, cols_a = (m, k) if ta == OP_N else (k, m)
            rows_b, cols_b = (k, n) if tb == OP_N else (n, k)
            for which, (typ, rows, cols, ld, stride) in enumerate(((type_a, rows_a, cols_a, lda, stride_a), (type_b, rows_b, cols_b, ldb, stride_b),
                                                                   (type_c, m, n, ldc, stride_c), (type_d, m, n, ldd, stride_d))):
                layout = _vp()
                status = lib.cublasLtMatrixLayoutCreate(C.byref(layout), typ, rows, cols, ld)
                if status:
                    raise BlasError("cublasLtMatrixLayoutCreate", status)
                layouts.append(layout)
                self._set(lib.cublasLtMatrixLayoutSetAttribute, layout, LT_LAYOUT_BATCH_COUNT, C.c_int32, batch)
                self._set(lib.cublasLtMatrixLayoutSetAttribute, layout, LT_LAYOUT_BATCH_STRIDE, C.c_int64, stride)
                if orders[which] is not None:
                    self._set(lib.cublasLtMatrixLayoutSetAttribute, layout, LT_LAYOUT_ORDER, C.c_int32, orders[which])
            a = C.create_string_buffer(pack_scalar(alpha, compute), 8)
            b = C.create_string_buffer(pack_scalar(beta, compute), 8)
            heuristic = C.create_string_buffer(96)
            found = _i(0)
            status = lib.cublasLtMatmulAlgoGetHeuristic(self.handle, desc, layouts[0], layouts[1], layouts[2], layouts[3], None, 1,
                                                        C.addressof(heuristic), C.byref(found))
            if status == 0 and found.value == 1:
                status = lib.cublasLtMatmul(self.handle, desc, C.addressof(a), A, layouts[0], B, layouts[1], C.addressof(b), Cp,
                                            layouts[2], D, layouts[3], C.addressof(heuristic), None, 0, stream)
            if check and status:
                raise BlasError("cublasLtMatmul", status)
            return status
        finally:
            for layout in layouts:
                lib.cublasLtMatrixLayoutDestroy(layout)
            lib.cublasLtMatmulDescDestroy(desc)

    def last_path(self) -> int:
        return self.lib.vkzbLastPath()

    def launch_count(self) -> int:
        return self.lib.vkzbLaunchCount()

    def set_output_mirrors(self, local_base: int, nbytes: int, mirrors: list[int]):
        """Every later GEMM on this handle whose result lies in [local_base, local_base + nbytes) also writes it, tile by
        tile, to the same offset in the `mirrors` buffers (extension vkzbSetOutputMirrors); an empty list switches it off."""
        arr = (_vp * max(1, len(mirrors)))(*mirrors)
        status = self.lib.vkzbSetOutputMirrors(self.handle, local_base, nbytes, len(mirrors), arr)
        if status:
            raise BlasError("vkzbSetOutputMirrors", status)
