// libcublasLt.so.12 entry points: descriptors, the one-algorithm heuristic, and cublasLtMatmul.
//
// Same surface and status behaviour as k0zi/Vulkanizer's src/cublas/cublasLt.cpp (:15-37 descriptors, :80-87 what is
// supported, :137-331 attribute plumbing, :333-416 matmul). The matmul itself is built differently: bias, ReLU and
// GELU are applied in the GEMM kernel's epilogue and C is read where it lies, so there is neither a copy of C into
// D (cublasLt.cpp:363-378) nor a second pass over D (cublasLt.cpp:386-412), and the handle's own stream and pointer
// mode are never touched (cublasLt.cpp:354-359 retargets them for the duration of the call).
#include <algorithm>
#include <cstring>
#include <new>

#define VKZB_HAVE_CUDA_TYPES
#include <library_types.h>

#include "../../include/vkzb_cublaslt.h"
#include "../../include/vkzb_ext.h"
#include "blas_internal.h"

struct cublasLtMatmulDescOpaque_st {
    cublasComputeType_t compute = CUBLAS_COMPUTE_32F;
    cudaDataType scaleType = CUDA_R_32F;
    int32_t pointerMode = CUBLASLT_POINTER_MODE_HOST;
    int32_t transa = CUBLAS_OP_N, transb = CUBLAS_OP_N, transc = CUBLAS_OP_N;
    uint32_t epilogue = CUBLASLT_EPILOGUE_DEFAULT;
    const void* bias = nullptr;
    int64_t biasBatchStride = 0;
    int32_t biasType = -1;  // -1: the type of D
};

struct cublasLtMatrixLayoutOpaque_st {
    cudaDataType type = CUDA_R_32F;
    int32_t order = CUBLASLT_ORDER_COL;
    uint64_t rows = 0, cols = 0;
    int64_t ld = 0;
    int32_t batchCount = 1;
    int64_t batchStride = 0;
};

struct cublasLtMatmulPreferenceOpaque_st {
    uint64_t maxWorkspace = 0;
};

namespace {

using namespace vkzb;

bool epilogueParts(uint32_t epilogue, bool& bias, int& activation) {
    switch (epilogue) {
    case CUBLASLT_EPILOGUE_DEFAULT: bias = false, activation = kActNone; return true;
    case CUBLASLT_EPILOGUE_RELU: bias = false, activation = kActRelu; return true;
    case CUBLASLT_EPILOGUE_BIAS: bias = true, activation = kActNone; return true;
    case CUBLASLT_EPILOGUE_RELU_BIAS: bias = true, activation = kActRelu; return true;
    case CUBLASLT_EPILOGUE_GELU: bias = false, activation = kActGelu; return true;
    case CUBLASLT_EPILOGUE_GELU_BIAS: bias = true, activation = kActGelu; return true;
    default: return false;  // aux outputs and gradients
    }
}

bool floatType(int t) { return t == kF32 || t == kF16 || t == kBF16; }

// What cublasLtMatmul serves; the heuristic and the algorithm check answer with the same predicate.
bool supported(const cublasLtMatmulDescOpaque_st& d, const cublasLtMatrixLayoutOpaque_st* const (&layouts)[4]) {
    for (const auto* l : layouts)
        if (!l || l->order != CUBLASLT_ORDER_COL || dtypeOf(l->type) == kBadType) return false;
    const int ta = dtypeOf(layouts[0]->type), tb = dtypeOf(layouts[1]->type), tc = dtypeOf(layouts[2]->type),
              td = dtypeOf(layouts[3]->type);
    const int st = scalarTypeOf(d.compute);
    const bool floats = floatType(ta) && floatType(tb) && floatType(tc) && floatType(td) && st == kScalarF32;
    const bool ints = ta == kS8 && tb == kS8 && tc == kS32 && td == kS32 && st == kScalarS32;
    if (!floats && !ints) return false;
    bool bias;
    int activation;
    if (d.transc != CUBLAS_OP_N || !epilogueParts(d.epilogue, bias, activation)) return false;
    if (ints && (bias || activation != kActNone)) return false;
    if (d.biasType >= 0 && !floatType(dtypeOf(cudaDataType(d.biasType)))) return false;
    return d.pointerMode == CUBLASLT_POINTER_MODE_HOST || d.pointerMode == CUBLASLT_POINTER_MODE_DEVICE;
}

template <class T>
cublasStatus_t setField(T& field, const void* buf, size_t size) {
    if (!buf || size != sizeof(T)) return CUBLAS_STATUS_INVALID_VALUE;
    std::memcpy(&field, buf, sizeof(T));
    return CUBLAS_STATUS_SUCCESS;
}

template <class T>
cublasStatus_t getField(const T& field, void* buf, size_t size, size_t* written) {
    if (written) *written = sizeof(T);
    if (!buf && size == 0) return written ? CUBLAS_STATUS_SUCCESS : CUBLAS_STATUS_INVALID_VALUE;
    if (!buf || size < sizeof(T)) return CUBLAS_STATUS_INVALID_VALUE;
    std::memcpy(buf, &field, sizeof(T));
    return CUBLAS_STATUS_SUCCESS;
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

cublasStatus_t cublasLtCreate(cublasLtHandle_t* lightHandle) {
    if (!lightHandle) return CUBLAS_STATUS_INVALID_VALUE;
    if (cudaFree(nullptr) != cudaSuccess) return CUBLAS_STATUS_NOT_INITIALIZED;
    auto* h = new (std::nothrow) cublasContext;
    if (!h) return CUBLAS_STATUS_ALLOC_FAILED;
    cudaGetDevice(&h->device);
    *lightHandle = h;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtDestroy(cublasLtHandle_t lightHandle) {
    if (!lightHandle) return CUBLAS_STATUS_NOT_INITIALIZED;
    if (lightHandle->scratch) cudaFree(lightHandle->scratch);
    delete lightHandle;
    return CUBLAS_STATUS_SUCCESS;
}

size_t cublasLtGetVersion(void) { return VKZB_CUBLAS_VERSION; }
size_t cublasLtGetCudartVersion(void) { return CUDART_VERSION; }

cublasStatus_t cublasLtMatmulDescCreate(cublasLtMatmulDesc_t* matmulDesc, cublasComputeType_t computeType, cudaDataType scaleType) {
    if (!matmulDesc) return CUBLAS_STATUS_INVALID_VALUE;
    auto* d = new (std::nothrow) cublasLtMatmulDescOpaque_st;
    if (!d) return CUBLAS_STATUS_ALLOC_FAILED;
    d->compute = computeType;
    d->scaleType = scaleType;
    *matmulDesc = d;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatmulDescDestroy(cublasLtMatmulDesc_t matmulDesc) {
    delete matmulDesc;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatmulDescSetAttribute(cublasLtMatmulDesc_t d, cublasLtMatmulDescAttributes_t attr, const void* buf,
                                              size_t size) {
    if (!d) return CUBLAS_STATUS_INVALID_VALUE;
    switch (int(attr)) {
    case CUBLASLT_MATMUL_DESC_COMPUTE_TYPE: return setField(d->compute, buf, size);
    case CUBLASLT_MATMUL_DESC_SCALE_TYPE: return setField(d->scaleType, buf, size);
    case CUBLASLT_MATMUL_DESC_POINTER_MODE: return setField(d->pointerMode, buf, size);
    case CUBLASLT_MATMUL_DESC_TRANSA: return setField(d->transa, buf, size);
    case CUBLASLT_MATMUL_DESC_TRANSB: return setField(d->transb, buf, size);
    case CUBLASLT_MATMUL_DESC_TRANSC: return setField(d->transc, buf, size);
    case CUBLASLT_MATMUL_DESC_EPILOGUE: return setField(d->epilogue, buf, size);
    case CUBLASLT_MATMUL_DESC_BIAS_POINTER: return setField(d->bias, buf, size);
    case CUBLASLT_MATMUL_DESC_BIAS_BATCH_STRIDE: return setField(d->biasBatchStride, buf, size);
    case CUBLASLT_MATMUL_DESC_BIAS_DATA_TYPE: return setField(d->biasType, buf, size);
    // hints that change nothing here
    case CUBLASLT_MATMUL_DESC_SM_COUNT_TARGET:
    case CUBLASLT_MATMUL_DESC_FAST_ACCUM:
    case CUBLASLT_MATMUL_DESC_FILL_MODE: return buf ? CUBLAS_STATUS_SUCCESS : CUBLAS_STATUS_INVALID_VALUE;
    default: return CUBLAS_STATUS_NOT_SUPPORTED;
    }
}

cublasStatus_t cublasLtMatmulDescGetAttribute(cublasLtMatmulDesc_t d, cublasLtMatmulDescAttributes_t attr, void* buf,
                                              size_t size, size_t* written) {
    if (!d) return CUBLAS_STATUS_INVALID_VALUE;
    switch (int(attr)) {
    case CUBLASLT_MATMUL_DESC_COMPUTE_TYPE: return getField(d->compute, buf, size, written);
    case CUBLASLT_MATMUL_DESC_SCALE_TYPE: return getField(d->scaleType, buf, size, written);
    case CUBLASLT_MATMUL_DESC_POINTER_MODE: return getField(d->pointerMode, buf, size, written);
    case CUBLASLT_MATMUL_DESC_TRANSA: return getField(d->transa, buf, size, written);
    case CUBLASLT_MATMUL_DESC_TRANSB: return getField(d->transb, buf, size, written);
    case CUBLASLT_MATMUL_DESC_TRANSC: return getField(d->transc, buf, size, written);
    case CUBLASLT_MATMUL_DESC_EPILOGUE: return getField(d->epilogue, buf, size, written);
    case CUBLASLT_MATMUL_DESC_BIAS_POINTER: return getField(d->bias, buf, size, written);
    case CUBLASLT_MATMUL_DESC_BIAS_BATCH_STRIDE: return getField(d->biasBatchStride, buf, size, written);
    case CUBLASLT_MATMUL_DESC_BIAS_DATA_TYPE: return getField(d->biasType, buf, size, written);
    default: return CUBLAS_STATUS_NOT_SUPPORTED;
    }
}

cublasStatus_t cublasLtMatrixLayoutCreate(cublasLtMatrixLayout_t* matLayout, cudaDataType type, uint64_t rows, uint64_t cols,
                                          int64_t ld) {
    if (!matLayout) return CUBLAS_STATUS_INVALID_VALUE;
    auto* l = new (std::nothrow) cublasLtMatrixLayoutOpaque_st;
    if (!l) return CUBLAS_STATUS_ALLOC_FAILED;
    l->type = type, l->rows = rows, l->cols = cols, l->ld = ld;
    *matLayout = l;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatrixLayoutDestroy(cublasLtMatrixLayout_t matLayout) {
    delete matLayout;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatrixLayoutSetAttribute(cublasLtMatrixLayout_t l, cublasLtMatrixLayoutAttribute_t attr, const void* buf,
                                                size_t size) {
    if (!l) return CUBLAS_STATUS_INVALID_VALUE;
    switch (int(attr)) {
    case CUBLASLT_MATRIX_LAYOUT_TYPE: return setField(l->type, buf, size);
    case CUBLASLT_MATRIX_LAYOUT_ORDER: return setField(l->order, buf, size);
    case CUBLASLT_MATRIX_LAYOUT_ROWS: return setField(l->rows, buf, size);
    case CUBLASLT_MATRIX_LAYOUT_COLS: return setField(l->cols, buf, size);
    case CUBLASLT_MATRIX_LAYOUT_LD: return setField(l->ld, buf, size);
    case CUBLASLT_MATRIX_LAYOUT_BATCH_COUNT: return setField(l->batchCount, buf, size);
    case CUBLASLT_MATRIX_LAYOUT_STRIDED_BATCH_OFFSET: return setField(l->batchStride, buf, size);
    default: return CUBLAS_STATUS_NOT_SUPPORTED;
    }
}

cublasStatus_t cublasLtMatrixLayoutGetAttribute(cublasLtMatrixLayout_t l, cublasLtMatrixLayoutAttribute_t attr, void* buf,
                                                size_t size, size_t* written) {
    if (!l) return CUBLAS_STATUS_INVALID_VALUE;
    switch (int(attr)) {
    case CUBLASLT_MATRIX_LAYOUT_TYPE: return getField(l->type, buf, size, written);
    case CUBLASLT_MATRIX_LAYOUT_ORDER: return getField(l->order, buf, size, written);
    case CUBLASLT_MATRIX_LAYOUT_ROWS: return getField(l->rows, buf, size, written);
    case CUBLASLT_MATRIX_LAYOUT_COLS: return getField(l->cols, buf, size, written);
    case CUBLASLT_MATRIX_LAYOUT_LD: return getField(l->ld, buf, size, written);
    case CUBLASLT_MATRIX_LAYOUT_BATCH_COUNT: return getField(l->batchCount, buf, size, written);
    case CUBLASLT_MATRIX_LAYOUT_STRIDED_BATCH_OFFSET: return getField(l->batchStride, buf, size, written);
    default: return CUBLAS_STATUS_NOT_SUPPORTED;
    }
}

cublasStatus_t cublasLtMatmulPreferenceCreate(cublasLtMatmulPreference_t* pref) {
    if (!pref) return CUBLAS_STATUS_INVALID_VALUE;
    *pref = new (std::nothrow) cublasLtMatmulPreferenceOpaque_st;
    return *pref ? CUBLAS_STATUS_SUCCESS : CUBLAS_STATUS_ALLOC_FAILED;
}

cublasStatus_t cublasLtMatmulPreferenceDestroy(cublasLtMatmulPreference_t pref) {
    delete pref;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatmulPreferenceSetAttribute(cublasLtMatmulPreference_t pref, cublasLtMatmulPreferenceAttributes_t attr,
                                                    const void* buf, size_t size) {
    if (!pref || !buf) return CUBLAS_STATUS_INVALID_VALUE;
    if (attr == CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES) return setField(pref->maxWorkspace, buf, size);
    return CUBLAS_STATUS_SUCCESS;  // search mode, alignments, waves: every request is served the same way
}

cublasStatus_t cublasLtMatmulPreferenceGetAttribute(cublasLtMatmulPreference_t pref, cublasLtMatmulPreferenceAttributes_t attr,
                                                    void* buf, size_t size, size_t* written) {
    if (!pref) return CUBLAS_STATUS_INVALID_VALUE;
    if (attr == CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES) return getField(pref->maxWorkspace, buf, size, written);
    return CUBLAS_STATUS_NOT_SUPPORTED;
}

cublasStatus_t cublasLtMatmulAlgoGetHeuristic(cublasLtHandle_t h, cublasLtMatmulDesc_t desc, cublasLtMatrixLayout_t Adesc,
                                              cublasLtMatrixLayout_t Bdesc, cublasLtMatrixLayout_t Cdesc,
                                              cublasLtMatrixLayout_t Ddesc, cublasLtMatmulPreference_t, int requested,
                                              cublasLtMatmulHeuristicResult_t results[], int* returned) {
    if (!h || !desc || requested < 1 || !results || !returned) return CUBLAS_STATUS_INVALID_VALUE;
    *returned = 0;
    const cublasLtMatrixLayoutOpaque_st* const layouts[4] = {Adesc, Bdesc, Cdesc, Ddesc};
    if (!supported(*desc, layouts)) return CUBLAS_STATUS_NOT_SUPPORTED;
    results[0] = {};
    results[0].workspaceSize = 0;
    results[0].state = CUBLAS_STATUS_SUCCESS;
    results[0].wavesCount = 1.0f;
    *returned = 1;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatmulAlgoInit(cublasLtHandle_t h, cublasComputeType_t, cudaDataType, cudaDataType, cudaDataType,
                                      cudaDataType, cudaDataType, int, cublasLtMatmulAlgo_t* algo) {
    if (!h || !algo) return CUBLAS_STATUS_INVALID_VALUE;
    *algo = {};
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatmulAlgoCheck(cublasLtHandle_t h, cublasLtMatmulDesc_t desc, cublasLtMatrixLayout_t Adesc,
                                       cublasLtMatrixLayout_t Bdesc, cublasLtMatrixLayout_t Cdesc, cublasLtMatrixLayout_t Ddesc,
                                       const cublasLtMatmulAlgo_t* algo, cublasLtMatmulHeuristicResult_t* result) {
    if (!h || !desc || !algo || !result) return CUBLAS_STATUS_INVALID_VALUE;
    const cublasLtMatrixLayoutOpaque_st* const layouts[4] = {Adesc, Bdesc, Cdesc, Ddesc};
    if (!supported(*desc, layouts)) return CUBLAS_STATUS_NOT_SUPPORTED;
    *result = {};
    result->algo = *algo;
    result->state = CUBLAS_STATUS_SUCCESS;
    result->wavesCount = 1.0f;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatmulAlgoConfigSetAttribute(cublasLtMatmulAlgo_t* algo, int, const void* buf, size_t) {
    return algo && buf ? CUBLAS_STATUS_SUCCESS : CUBLAS_STATUS_INVALID_VALUE;
}

cublasStatus_t cublasLtMatmulAlgoConfigGetAttribute(const cublasLtMatmulAlgo_t* algo, int, void* buf, size_t size,
                                                    size_t* written) {
    if (!algo) return CUBLAS_STATUS_INVALID_VALUE;
    if (buf) std::memset(buf, 0, size);  // ids, tiles, stages, splits: all zero
    if (written) *written = size;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatmul(cublasLtHandle_t h, cublasLtMatmulDesc_t desc, const void* alpha, const void* A,
                              cublasLtMatrixLayout_t Adesc, const void* B, cublasLtMatrixLayout_t Bdesc, const void* beta,
                              const void* C, cublasLtMatrixLayout_t Cdesc, void* D, cublasLtMatrixLayout_t Ddesc,
                              const cublasLtMatmulAlgo_t*, void*, size_t, cudaStream_t stream) {
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    if (!desc || !Adesc || !Bdesc || !Cdesc || !Ddesc || !alpha || !beta) return CUBLAS_STATUS_INVALID_VALUE;
    const cublasLtMatrixLayoutOpaque_st* const layouts[4] = {Adesc, Bdesc, Cdesc, Ddesc};
    if (!supported(*desc, layouts)) return CUBLAS_STATUS_NOT_SUPPORTED;
    if (Cdesc->rows != Ddesc->rows || Cdesc->cols != Ddesc->cols) return CUBLAS_STATUS_INVALID_VALUE;
    const bool ta = desc->transa != CUBLAS_OP_N, tb = desc->transb != CUBLAS_OP_N;
    if (Ddesc->rows > INT32_MAX || Ddesc->cols > INT32_MAX || Adesc->rows > INT32_MAX || Adesc->cols > INT32_MAX)
        return CUBLAS_STATUS_NOT_SUPPORTED;

    Problem p;
    p.transA = ta, p.transB = tb;
    p.m = int(Ddesc->rows), p.n = int(Ddesc->cols);
    p.k = int(ta ? Adesc->rows : Adesc->cols);
    p.batch = std::max(1, Ddesc->batchCount);
    const int rowsA = ta ? p.k : p.m, rowsB = tb ? p.n : p.k;
    if (Adesc->ld < std::max(1, rowsA) || Bdesc->ld < std::max(1, rowsB) || Cdesc->ld < std::max(1, p.m) ||
        Ddesc->ld < std::max(1, p.m))
        return CUBLAS_STATUS_INVALID_VALUE;
    if (p.m == 0 || p.n == 0) return CUBLAS_STATUS_SUCCESS;
    p.A = A, p.B = B;
    p.typeA = dtypeOf(Adesc->type), p.typeB = dtypeOf(Bdesc->type);
    p.lda = Adesc->ld, p.ldb = Bdesc->ld;
    p.strideA = Adesc->batchCount > 1 ? Adesc->batchStride : 0;
    p.strideB = Bdesc->batchCount > 1 ? Bdesc->batchStride : 0;
    const int st = scalarTypeOf(desc->compute);
    p.accType = st == kScalarS32 ? kS32 : kF32;
    p.allowTf32 = h->math == CUBLAS_TF32_TENSOR_OP_MATH || desc->compute == CUBLAS_COMPUTE_32F_FAST_TF32;

    bool bias;
    int activation;
    epilogueParts(desc->epilogue, bias, activation);
    if (bias && !desc->bias) return CUBLAS_STATUS_INVALID_VALUE;
    EpilogueArgs& e = p.epi;
    e.D = D, e.C = C;
    e.ldd = Ddesc->ld, e.ldc = Cdesc->ld;
    e.strideD = Ddesc->batchStride;
    e.strideC = Cdesc->batchCount > 1 ? Cdesc->batchStride : 0;
    e.typeD = dtypeOf(Ddesc->type), e.typeC = dtypeOf(Cdesc->type);
    e.bias = bias ? desc->bias : nullptr;
    e.biasStride = desc->biasBatchStride;
    e.typeBias = desc->biasType >= 0 ? dtypeOf(cudaDataType(desc->biasType)) : e.typeD;
    e.activation = activation;
    // Where the reference runs its epilogue as a second pass, D has already been rounded to its storage
    // type once (tests/cublas.cpp:467 of the reference expects exactly that); the fused epilogue rounds at the same point.
    e.roundBeforeBias = (bias || activation != kActNone) && e.typeD != kF32;
    e.pointerArrays = 0;
    if (!fillScalars(e.scalars, alpha, beta, st, desc->pointerMode == CUBLASLT_POINTER_MODE_DEVICE))
        return CUBLAS_STATUS_INVALID_VALUE;

    cublasContext call = *h;  // the handle itself stays as it is: only this call runs on `stream`
    call.scratch = nullptr, call.scratchBytes = 0;  // a light handle carries no split-k scratch (its products are not split)
    call.stream = stream;
    return dispatch(&call, p);
}

// cuBLASLt 13's grouped layouts: not served (arguments ignored).
cublasStatus_t cublasLtGroupedMatrixLayoutCreate() { return CUBLAS_STATUS_NOT_SUPPORTED; }

}  // extern "C"
#pragma GCC visibility pop
