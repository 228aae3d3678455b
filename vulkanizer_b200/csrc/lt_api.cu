// libcublasLt.so.12 entry points: descriptors, the one-algorithm heuristic, and cublasLtMatmul.
//
// Same exported surface and status behaviour as k0zi/Vulkanizer's src/cublas/cublasLt.cpp (:137-331 descriptor calls,
// :333-416 matmul), built differently throughout:
//   * a descriptor is a bag of 8-byte slots indexed by NVIDIA's attribute number, and ONE table per descriptor kind says
//     which numbers exist, how many bytes each carries and whether it is only a hint; a single routine walks the table for
//     every Set / Get call;
//   * the matmul applies bias, ReLU and GELU inside the GEMM kernel's epilogue and reads C where it lies: no copy of C
//     into D (cublasLt.cpp:363-378), no second pass over D (:386-412), and the handle is never retargeted (:354-359);
//   * it serves what the reference refuses (cublasLt.cpp:68-78, 83): the epilogues with an auxiliary matrix (RELU_AUX,
//     GELU_AUX and their BIAS forms), the backward epilogues (DRELU, DGELU, with or without BGRAD), the bias gradients of
//     the operands (BGRADA, BGRADB), and matrices in row order (CUBLASLT_ORDER_ROW) by running the transposed problem.
#include <algorithm>
#include <cstring>
#include <new>

#define VKZB_HAVE_CUDA_TYPES
#include <library_types.h>

#include "../../include/vkzb_cublaslt.h"
#include "../../include/vkzb_ext.h"
#include "blas_internal.h"

namespace {

constexpr int kSlots = 32;  // attribute numbers in use stay below this

// One row of an attribute table: NVIDIA's attribute number, the size its value must have, and whether the value matters
// here (a hint is accepted and forgotten).
struct AttributeRow {
    int number;
    unsigned bytes;
    bool hint;
};

struct AttributeBag {
    uint64_t slot[kSlots] = {};

    template <class T>
    T as(int number) const {
        T v;
        std::memcpy(&v, &slot[number], sizeof v);
        return v;
    }
    template <class T>
    void put(int number, T v) {
        slot[number] = 0;
        std::memcpy(&slot[number], &v, sizeof v);
    }
};

template <size_t N>
const AttributeRow* findRow(const AttributeRow (&table)[N], int number) {
    for (const AttributeRow& row : table)
        if (row.number == number) return &row;
    return nullptr;
}

// Set: the buffer must hold exactly the attribute's size. Unknown numbers are NOT_SUPPORTED, hints succeed untouched.
template <size_t N>
cublasStatus_t writeAttribute(AttributeBag* bag, const AttributeRow (&table)[N], int number, const void* buf, size_t size) {
    if (!bag) return CUBLAS_STATUS_INVALID_VALUE;
    const AttributeRow* row = findRow(table, number);
    if (!row) return CUBLAS_STATUS_NOT_SUPPORTED;
    if (!buf) return CUBLAS_STATUS_INVALID_VALUE;
    if (row->hint) return CUBLAS_STATUS_SUCCESS;
    if (size != row->bytes) return CUBLAS_STATUS_INVALID_VALUE;
    bag->slot[number] = 0;
    std::memcpy(&bag->slot[number], buf, row->bytes);
    return CUBLAS_STATUS_SUCCESS;
}

// Get: a null buffer of size 0 asks for the size only; hints cannot be read back.
template <size_t N>
cublasStatus_t readAttribute(const AttributeBag* bag, const AttributeRow (&table)[N], int number, void* buf, size_t size, size_t* written) {
    if (!bag) return CUBLAS_STATUS_INVALID_VALUE;
    const AttributeRow* row = findRow(table, number);
    if (!row || row->hint) return CUBLAS_STATUS_NOT_SUPPORTED;
    if (written) *written = row->bytes;
    if (!buf && size == 0) return written ? CUBLAS_STATUS_SUCCESS : CUBLAS_STATUS_INVALID_VALUE;
    if (!buf || size < row->bytes) return CUBLAS_STATUS_INVALID_VALUE;
    std::memcpy(buf, &bag->slot[number], row->bytes);
    return CUBLAS_STATUS_SUCCESS;
}

constexpr AttributeRow kMatmulRows[] = {
    {CUBLASLT_MATMUL_DESC_COMPUTE_TYPE, 4, false},        {CUBLASLT_MATMUL_DESC_SCALE_TYPE, 4, false},
    {CUBLASLT_MATMUL_DESC_POINTER_MODE, 4, false},        {CUBLASLT_MATMUL_DESC_TRANSA, 4, false},
    {CUBLASLT_MATMUL_DESC_TRANSB, 4, false},              {CUBLASLT_MATMUL_DESC_TRANSC, 4, false},
    {CUBLASLT_MATMUL_DESC_EPILOGUE, 4, false},            {CUBLASLT_MATMUL_DESC_BIAS_POINTER, 8, false},
    {CUBLASLT_MATMUL_DESC_BIAS_BATCH_STRIDE, 8, false},   {CUBLASLT_MATMUL_DESC_BIAS_DATA_TYPE, 4, false},
    {CUBLASLT_MATMUL_DESC_EPILOGUE_AUX_POINTER, 8, false}, {CUBLASLT_MATMUL_DESC_EPILOGUE_AUX_LD, 8, false},
    {CUBLASLT_MATMUL_DESC_EPILOGUE_AUX_BATCH_STRIDE, 8, false}, {CUBLASLT_MATMUL_DESC_EPILOGUE_AUX_DATA_TYPE, 4, false},
    {CUBLASLT_MATMUL_DESC_SM_COUNT_TARGET, 4, true},      {CUBLASLT_MATMUL_DESC_FAST_ACCUM, 1, true},
    {CUBLASLT_MATMUL_DESC_FILL_MODE, 4, true},
};
constexpr AttributeRow kLayoutRows[] = {
    {CUBLASLT_MATRIX_LAYOUT_TYPE, 4, false}, {CUBLASLT_MATRIX_LAYOUT_ORDER, 4, false}, {CUBLASLT_MATRIX_LAYOUT_ROWS, 8, false},
    {CUBLASLT_MATRIX_LAYOUT_COLS, 8, false}, {CUBLASLT_MATRIX_LAYOUT_LD, 8, false},    {CUBLASLT_MATRIX_LAYOUT_BATCH_COUNT, 4, false},
    {CUBLASLT_MATRIX_LAYOUT_STRIDED_BATCH_OFFSET, 8, false},
};
constexpr AttributeRow kPreferenceRows[] = {{CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, 8, false}};

constexpr int kBiasTypeUnset = -1;  // bias (and auxiliary) type not given: the type of D

}  // namespace

struct cublasLtMatmulDescOpaque_st : AttributeBag {};
struct cublasLtMatrixLayoutOpaque_st : AttributeBag {};
struct cublasLtMatmulPreferenceOpaque_st : AttributeBag {};

namespace {

using namespace vkzb;

// A layout as cublasLtMatmul reads it.
struct LayoutView {
    int type;  // DType, or kBadType
    bool rowOrder, orderKnown;
    uint64_t rows, cols;
    int64_t ld;
    int batch;
    int64_t batchStride;
};

LayoutView viewOf(const cublasLtMatrixLayoutOpaque_st& l) {
    LayoutView v;
    v.type = dtypeOf(cudaDataType(l.as<int32_t>(CUBLASLT_MATRIX_LAYOUT_TYPE)));
    const int32_t order = l.as<int32_t>(CUBLASLT_MATRIX_LAYOUT_ORDER);
    v.orderKnown = order == CUBLASLT_ORDER_COL || order == CUBLASLT_ORDER_ROW;
    v.rowOrder = order == CUBLASLT_ORDER_ROW;
    v.rows = l.as<uint64_t>(CUBLASLT_MATRIX_LAYOUT_ROWS), v.cols = l.as<uint64_t>(CUBLASLT_MATRIX_LAYOUT_COLS);
    v.ld = l.as<int64_t>(CUBLASLT_MATRIX_LAYOUT_LD);
    v.batch = l.as<int32_t>(CUBLASLT_MATRIX_LAYOUT_BATCH_COUNT);
    v.batchStride = l.as<int64_t>(CUBLASLT_MATRIX_LAYOUT_STRIDED_BATCH_OFFSET);
    return v;
}

// An epilogue number taken apart.
struct EpiloguePlan {
    bool known = true;
    bool bias = false;        // a bias vector is added
    int activation = kActNone;
    int auxMode = kAuxNone;
    int gradient = 0;         // 0 none, 1 sum of op(A) over k (BGRADA), 2 sum of op(B) over k (BGRADB), 3 sum of D over its columns
};

EpiloguePlan planOf(uint32_t epilogue) {
    // NVIDIA's numbers are sums of flags: 2 ReLU, 4 bias, 8 ReLU', 16 bias gradient of D, 32 GELU, 64 GELU', 128 auxiliary
    // matrix, 256 / 512 bias gradient of A / B; only the combinations NVIDIA names are accepted.
    EpiloguePlan e;
    const auto with = [&](bool bias, int activation, int auxMode, int gradient) {
        e.bias = bias, e.activation = activation, e.auxMode = auxMode, e.gradient = gradient;
    };
    switch (epilogue) {
    case CUBLASLT_EPILOGUE_DEFAULT: break;
    case CUBLASLT_EPILOGUE_BIAS: with(true, kActNone, kAuxNone, 0); break;
    case CUBLASLT_EPILOGUE_RELU: with(false, kActRelu, kAuxNone, 0); break;
    case CUBLASLT_EPILOGUE_RELU_BIAS: with(true, kActRelu, kAuxNone, 0); break;
    case CUBLASLT_EPILOGUE_GELU: with(false, kActGelu, kAuxNone, 0); break;
    case CUBLASLT_EPILOGUE_GELU_BIAS: with(true, kActGelu, kAuxNone, 0); break;
    case CUBLASLT_EPILOGUE_RELU_AUX: with(false, kActRelu, kAuxWriteMask, 0); break;
    case CUBLASLT_EPILOGUE_RELU_AUX_BIAS: with(true, kActRelu, kAuxWriteMask, 0); break;
    case CUBLASLT_EPILOGUE_GELU_AUX: with(false, kActGelu, kAuxWriteInput, 0); break;
    case CUBLASLT_EPILOGUE_GELU_AUX_BIAS: with(true, kActGelu, kAuxWriteInput, 0); break;
    case CUBLASLT_EPILOGUE_DRELU: with(false, kActDRelu, kAuxReadMask, 0); break;
    case CUBLASLT_EPILOGUE_DRELU_BGRAD: with(false, kActDRelu, kAuxReadMask, 3); break;
    case CUBLASLT_EPILOGUE_DGELU: with(false, kActDGelu, kAuxReadInput, 0); break;
    case CUBLASLT_EPILOGUE_DGELU_BGRAD: with(false, kActDGelu, kAuxReadInput, 3); break;
    case CUBLASLT_EPILOGUE_BGRADA: with(false, kActNone, kAuxNone, 1); break;
    case CUBLASLT_EPILOGUE_BGRADB: with(false, kActNone, kAuxNone, 2); break;
    default: e.known = false; break;
    }
    return e;
}

bool isFloatStorage(int t) { return t == kF32 || t == kF16 || t == kBF16; }

// Everything about a request that does not depend on the data pointers: the one predicate behind the heuristic, the
// algorithm check and the matmul, so the three always agree (cublasLt.cpp:289, 312, 342-346 keep them in step likewise).
cublasStatus_t examine(const cublasLtMatmulDescOpaque_st* desc, const cublasLtMatrixLayoutOpaque_st* const (&layouts)[4], LayoutView (&views)[4],
                       EpiloguePlan& plan) {
    if (!desc) return CUBLAS_STATUS_INVALID_VALUE;
    for (int i = 0; i < 4; ++i) {
        if (!layouts[i]) return CUBLAS_STATUS_INVALID_VALUE;
        views[i] = viewOf(*layouts[i]);
        if (views[i].type == kBadType || !views[i].orderKnown) return CUBLAS_STATUS_NOT_SUPPORTED;
    }
    const LayoutView &a = views[0], &b = views[1], &c = views[2], &d = views[3];
    const int scalar = scalarTypeOf(cublasComputeType_t(desc->as<int32_t>(CUBLASLT_MATMUL_DESC_COMPUTE_TYPE)));
    const bool floats = isFloatStorage(a.type) && isFloatStorage(b.type) && isFloatStorage(c.type) && isFloatStorage(d.type) && scalar == kScalarF32;
    const bool ints = a.type == kS8 && b.type == kS8 && c.type == kS32 && d.type == kS32 && scalar == kScalarS32;
    if (!floats && !ints) return CUBLAS_STATUS_NOT_SUPPORTED;
    if (desc->as<int32_t>(CUBLASLT_MATMUL_DESC_TRANSC) != CUBLAS_OP_N) return CUBLAS_STATUS_NOT_SUPPORTED;
    const int32_t pointerMode = desc->as<int32_t>(CUBLASLT_MATMUL_DESC_POINTER_MODE);
    if (pointerMode != CUBLASLT_POINTER_MODE_HOST && pointerMode != CUBLASLT_POINTER_MODE_DEVICE) return CUBLAS_STATUS_NOT_SUPPORTED;
    plan = planOf(desc->as<uint32_t>(CUBLASLT_MATMUL_DESC_EPILOGUE));
    if (!plan.known) return CUBLAS_STATUS_NOT_SUPPORTED;
    const bool plainEpilogue = !plan.bias && plan.activation == kActNone && plan.gradient == 0;
    if (ints && !plainEpilogue) return CUBLAS_STATUS_NOT_SUPPORTED;
    if (c.rowOrder != d.rowOrder) return CUBLAS_STATUS_NOT_SUPPORTED;
    if (d.rowOrder && plan.auxMode != kAuxNone) return CUBLAS_STATUS_NOT_SUPPORTED;  // auxiliary matrices: column order only
    const int32_t biasType = desc->as<int32_t>(CUBLASLT_MATMUL_DESC_BIAS_DATA_TYPE);
    if (biasType != kBiasTypeUnset && !isFloatStorage(dtypeOf(cudaDataType(biasType)))) return CUBLAS_STATUS_NOT_SUPPORTED;
    const int32_t auxType = desc->as<int32_t>(CUBLASLT_MATMUL_DESC_EPILOGUE_AUX_DATA_TYPE);
    if (auxType != kBiasTypeUnset && !isFloatStorage(dtypeOf(cudaDataType(auxType)))) return CUBLAS_STATUS_NOT_SUPPORTED;
    return CUBLAS_STATUS_SUCCESS;
}

void fillHeuristic(cublasLtMatmulHeuristicResult_t& r, const cublasLtMatmulAlgo_t* algo) {
    std::memset(&r, 0, sizeof r);
    if (algo) r.algo = *algo;
    r.state = CUBLAS_STATUS_SUCCESS;
    r.wavesCount = 1.0f;  // workspaceSize stays 0: the kernels keep their accumulators in TMEM
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
    releaseScratch(lightHandle);
    delete lightHandle;
    return CUBLAS_STATUS_SUCCESS;
}

size_t cublasLtGetVersion(void) { return VKZB_CUBLAS_VERSION; }
size_t cublasLtGetCudartVersion(void) { return CUDART_VERSION; }

cublasStatus_t cublasLtMatmulDescCreate(cublasLtMatmulDesc_t* matmulDesc, cublasComputeType_t computeType, cudaDataType scaleType) {
    if (!matmulDesc) return CUBLAS_STATUS_INVALID_VALUE;
    auto* d = new (std::nothrow) cublasLtMatmulDescOpaque_st;
    if (!d) return CUBLAS_STATUS_ALLOC_FAILED;
    d->put<int32_t>(CUBLASLT_MATMUL_DESC_COMPUTE_TYPE, computeType);
    d->put<int32_t>(CUBLASLT_MATMUL_DESC_SCALE_TYPE, scaleType);
    d->put<int32_t>(CUBLASLT_MATMUL_DESC_POINTER_MODE, CUBLASLT_POINTER_MODE_HOST);
    d->put<int32_t>(CUBLASLT_MATMUL_DESC_TRANSA, CUBLAS_OP_N);
    d->put<int32_t>(CUBLASLT_MATMUL_DESC_TRANSB, CUBLAS_OP_N);
    d->put<int32_t>(CUBLASLT_MATMUL_DESC_TRANSC, CUBLAS_OP_N);
    d->put<uint32_t>(CUBLASLT_MATMUL_DESC_EPILOGUE, CUBLASLT_EPILOGUE_DEFAULT);
    d->put<int32_t>(CUBLASLT_MATMUL_DESC_BIAS_DATA_TYPE, kBiasTypeUnset);
    d->put<int32_t>(CUBLASLT_MATMUL_DESC_EPILOGUE_AUX_DATA_TYPE, kBiasTypeUnset);
    *matmulDesc = d;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatmulDescDestroy(cublasLtMatmulDesc_t matmulDesc) {
    delete matmulDesc;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatmulDescSetAttribute(cublasLtMatmulDesc_t d, cublasLtMatmulDescAttributes_t attr, const void* buf, size_t size) {
    return writeAttribute(d, kMatmulRows, int(attr), buf, size);
}

cublasStatus_t cublasLtMatmulDescGetAttribute(cublasLtMatmulDesc_t d, cublasLtMatmulDescAttributes_t attr, void* buf, size_t size,
                                              size_t* written) {
    return readAttribute(d, kMatmulRows, int(attr), buf, size, written);
}

cublasStatus_t cublasLtMatrixLayoutCreate(cublasLtMatrixLayout_t* matLayout, cudaDataType type, uint64_t rows, uint64_t cols, int64_t ld) {
    if (!matLayout) return CUBLAS_STATUS_INVALID_VALUE;
    auto* l = new (std::nothrow) cublasLtMatrixLayoutOpaque_st;
    if (!l) return CUBLAS_STATUS_ALLOC_FAILED;
    l->put<int32_t>(CUBLASLT_MATRIX_LAYOUT_TYPE, type);
    l->put<int32_t>(CUBLASLT_MATRIX_LAYOUT_ORDER, CUBLASLT_ORDER_COL);
    l->put<uint64_t>(CUBLASLT_MATRIX_LAYOUT_ROWS, rows);
    l->put<uint64_t>(CUBLASLT_MATRIX_LAYOUT_COLS, cols);
    l->put<int64_t>(CUBLASLT_MATRIX_LAYOUT_LD, ld);
    l->put<int32_t>(CUBLASLT_MATRIX_LAYOUT_BATCH_COUNT, 1);
    *matLayout = l;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatrixLayoutDestroy(cublasLtMatrixLayout_t matLayout) {
    delete matLayout;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatrixLayoutSetAttribute(cublasLtMatrixLayout_t l, cublasLtMatrixLayoutAttribute_t attr, const void* buf, size_t size) {
    return writeAttribute(l, kLayoutRows, int(attr), buf, size);
}

cublasStatus_t cublasLtMatrixLayoutGetAttribute(cublasLtMatrixLayout_t l, cublasLtMatrixLayoutAttribute_t attr, void* buf, size_t size,
                                                size_t* written) {
    return readAttribute(l, kLayoutRows, int(attr), buf, size, written);
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

// Only the workspace limit is remembered; search mode, alignments and wave counts change nothing (one algorithm serves all).
cublasStatus_t cublasLtMatmulPreferenceSetAttribute(cublasLtMatmulPreference_t pref, cublasLtMatmulPreferenceAttributes_t attr, const void* buf,
                                                    size_t size) {
    if (!pref || !buf) return CUBLAS_STATUS_INVALID_VALUE;
    const cublasStatus_t s = writeAttribute(pref, kPreferenceRows, int(attr), buf, size);
    return s == CUBLAS_STATUS_NOT_SUPPORTED ? CUBLAS_STATUS_SUCCESS : s;
}

cublasStatus_t cublasLtMatmulPreferenceGetAttribute(cublasLtMatmulPreference_t pref, cublasLtMatmulPreferenceAttributes_t attr, void* buf,
                                                    size_t size, size_t* written) {
    return readAttribute(pref, kPreferenceRows, int(attr), buf, size, written);
}

cublasStatus_t cublasLtMatmulAlgoGetHeuristic(cublasLtHandle_t h, cublasLtMatmulDesc_t desc, cublasLtMatrixLayout_t Adesc,
                                              cublasLtMatrixLayout_t Bdesc, cublasLtMatrixLayout_t Cdesc, cublasLtMatrixLayout_t Ddesc,
                                              cublasLtMatmulPreference_t, int requested, cublasLtMatmulHeuristicResult_t results[],
                                              int* returned) {
    if (!h || !desc || requested < 1 || !results || !returned) return CUBLAS_STATUS_INVALID_VALUE;
    *returned = 0;
    const cublasLtMatrixLayoutOpaque_st* const layouts[4] = {Adesc, Bdesc, Cdesc, Ddesc};
    LayoutView views[4];
    EpiloguePlan plan;
    if (examine(desc, layouts, views, plan) != CUBLAS_STATUS_SUCCESS) return CUBLAS_STATUS_NOT_SUPPORTED;
    fillHeuristic(results[0], nullptr);
    *returned = 1;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatmulAlgoInit(cublasLtHandle_t h, cublasComputeType_t, cudaDataType, cudaDataType, cudaDataType, cudaDataType,
                                      cudaDataType, int, cublasLtMatmulAlgo_t* algo) {
    if (!h || !algo) return CUBLAS_STATUS_INVALID_VALUE;
    std::memset(algo, 0, sizeof *algo);
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatmulAlgoCheck(cublasLtHandle_t h, cublasLtMatmulDesc_t desc, cublasLtMatrixLayout_t Adesc, cublasLtMatrixLayout_t Bdesc,
                                       cublasLtMatrixLayout_t Cdesc, cublasLtMatrixLayout_t Ddesc, const cublasLtMatmulAlgo_t* algo,
                                       cublasLtMatmulHeuristicResult_t* result) {
    if (!h || !desc || !algo || !result) return CUBLAS_STATUS_INVALID_VALUE;
    const cublasLtMatrixLayoutOpaque_st* const layouts[4] = {Adesc, Bdesc, Cdesc, Ddesc};
    LayoutView views[4];
    EpiloguePlan plan;
    if (examine(desc, layouts, views, plan) != CUBLAS_STATUS_SUCCESS) return CUBLAS_STATUS_NOT_SUPPORTED;
    fillHeuristic(*result, algo);
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatmulAlgoConfigSetAttribute(cublasLtMatmulAlgo_t* algo, int, const void* buf, size_t) {
    return algo && buf ? CUBLAS_STATUS_SUCCESS : CUBLAS_STATUS_INVALID_VALUE;
}

// Tile ids, stages, split counts: the one algorithm reports zero for all of them.
cublasStatus_t cublasLtMatmulAlgoConfigGetAttribute(const cublasLtMatmulAlgo_t* algo, int, void* buf, size_t size, size_t* written) {
    if (!algo) return CUBLAS_STATUS_INVALID_VALUE;
    if (buf) std::memset(buf, 0, size);
    if (written) *written = size;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasLtMatmul(cublasLtHandle_t h, cublasLtMatmulDesc_t desc, const void* alpha, const void* A, cublasLtMatrixLayout_t Adesc,
                              const void* B, cublasLtMatrixLayout_t Bdesc, const void* beta, const void* C, cublasLtMatrixLayout_t Cdesc, void* D,
                              cublasLtMatrixLayout_t Ddesc, const cublasLtMatmulAlgo_t*, void*, size_t, cudaStream_t stream) {
    VKZB_API_SCOPE();
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    if (!desc || !Adesc || !Bdesc || !Cdesc || !Ddesc || !alpha || !beta) return CUBLAS_STATUS_INVALID_VALUE;
    const cublasLtMatrixLayoutOpaque_st* const layouts[4] = {Adesc, Bdesc, Cdesc, Ddesc};
    LayoutView views[4];
    EpiloguePlan plan;
    if (const cublasStatus_t s = examine(desc, layouts, views, plan); s != CUBLAS_STATUS_SUCCESS) return s;
    const LayoutView &la = views[0], &lb = views[1], &lc = views[2], &ld = views[3];
    if (lc.rows != ld.rows || lc.cols != ld.cols) return CUBLAS_STATUS_INVALID_VALUE;
    if (ld.rows > INT32_MAX || ld.cols > INT32_MAX || la.rows > INT32_MAX || la.cols > INT32_MAX) return CUBLAS_STATUS_NOT_SUPPORTED;

    // The problem as the caller states it: D (m x n) = op(A) (m x k) op(B) (k x n).
    const bool userTa = desc->as<int32_t>(CUBLASLT_MATMUL_DESC_TRANSA) != CUBLAS_OP_N, userTb = desc->as<int32_t>(CUBLASLT_MATMUL_DESC_TRANSB) != CUBLAS_OP_N;
    const int m = int(ld.rows), n = int(ld.cols), k = int(userTa ? la.rows : la.cols);
    const auto ldFloor = [](const LayoutView& v) { return int64_t(std::max<uint64_t>(1, v.rowOrder ? v.cols : v.rows)); };
    if (la.ld < ldFloor(la) || lb.ld < ldFloor(lb) || lc.ld < ldFloor(lc) || ld.ld < ldFloor(ld)) return CUBLAS_STATUS_INVALID_VALUE;
    if (m == 0 || n == 0) return CUBLAS_STATUS_SUCCESS;
    // A matrix in row order is its transpose in column order: the stored (column-major) operand carries the opposite flag.
    const bool ta = userTa != la.rowOrder, tb = userTb != lb.rowOrder;

    Problem p;
    p.k = k;
    p.batch = std::max(1, ld.batch);
    const int scalar = scalarTypeOf(cublasComputeType_t(desc->as<int32_t>(CUBLASLT_MATMUL_DESC_COMPUTE_TYPE)));
    p.accType = scalar == kScalarS32 ? kS32 : kF32;
    p.allowTf32 = h->math == CUBLAS_TF32_TENSOR_OP_MATH || desc->as<int32_t>(CUBLASLT_MATMUL_DESC_COMPUTE_TYPE) == CUBLAS_COMPUTE_32F_FAST_TF32;
    const long long strideA = la.batch > 1 ? la.batchStride : 0, strideB = lb.batch > 1 ? lb.batchStride : 0;
    if (!ld.rowOrder) {
        p.transA = ta, p.transB = tb, p.m = m, p.n = n;
        p.A = A, p.typeA = la.type, p.lda = la.ld, p.strideA = strideA;
        p.B = B, p.typeB = lb.type, p.ldb = lb.ld, p.strideB = strideB;
    } else {
        // D in row order is D^T in column order: D^T = op(B)^T op(A)^T, so the operands change places and flags
        p.transA = !tb, p.transB = !ta, p.m = n, p.n = m;
        p.A = B, p.typeA = lb.type, p.lda = lb.ld, p.strideA = strideB;
        p.B = A, p.typeB = la.type, p.ldb = la.ld, p.strideB = strideA;
    }

    EpilogueArgs& e = p.epi;
    e.D = D, e.C = C;
    e.ldd = ld.ld, e.ldc = lc.ld;
    e.strideD = ld.batchStride;
    e.strideC = lc.batch > 1 ? lc.batchStride : 0;
    e.typeD = ld.type, e.typeC = lc.type;
    e.pointerArrays = 0;
    const int32_t biasType = desc->as<int32_t>(CUBLASLT_MATMUL_DESC_BIAS_DATA_TYPE);
    const int typeBias = biasType == kBiasTypeUnset ? e.typeD : dtypeOf(cudaDataType(biasType));
    const void* biasPointer = desc->as<const void*>(CUBLASLT_MATMUL_DESC_BIAS_POINTER);
    const long long biasStride = desc->as<int64_t>(CUBLASLT_MATMUL_DESC_BIAS_BATCH_STRIDE);
    if ((plan.bias || plan.gradient) && !biasPointer) return CUBLAS_STATUS_INVALID_VALUE;
    e.bias = plan.bias ? biasPointer : nullptr;
    e.biasStride = biasStride;
    e.typeBias = typeBias;
    e.biasAlongN = ld.rowOrder ? 1 : 0;  // the bias belongs to D's rows, which are the transposed problem's columns
    e.activation = plan.activation;
    e.auxMode = plan.auxMode;
    if (plan.auxMode != kAuxNone) {
        e.aux = desc->as<void*>(CUBLASLT_MATMUL_DESC_EPILOGUE_AUX_POINTER);
        e.auxLd = desc->as<int64_t>(CUBLASLT_MATMUL_DESC_EPILOGUE_AUX_LD);
        e.auxStride = desc->as<int64_t>(CUBLASLT_MATMUL_DESC_EPILOGUE_AUX_BATCH_STRIDE);
        const int32_t auxType = desc->as<int32_t>(CUBLASLT_MATMUL_DESC_EPILOGUE_AUX_DATA_TYPE);
        e.typeAux = auxType == kBiasTypeUnset ? e.typeD : dtypeOf(cudaDataType(auxType));
        const bool mask = plan.auxMode == kAuxWriteMask || plan.auxMode == kAuxReadMask;
        // a mask's leading dimension counts bits and keeps every column on a 32-bit word (NVIDIA asks for multiples of 128)
        if (!e.aux || e.auxLd < m || (mask && (e.auxLd % 32 != 0 || e.auxStride % 32 != 0 || (reinterpret_cast<uintptr_t>(e.aux) & 3) != 0)))
            return CUBLAS_STATUS_INVALID_VALUE;
    }
    // Where the reference runs its epilogue as a second pass, D has already been rounded to its storage type once (its
    // acceptance test expects exactly that, tests/cublas.cpp:467); the fused forward epilogues round at the same point.
    const bool forward = plan.bias || plan.activation == kActRelu || plan.activation == kActGelu;
    e.roundBeforeBias = forward && e.typeD != kF32;
    if (!fillScalars(e.scalars, alpha, beta, scalar, desc->as<int32_t>(CUBLASLT_MATMUL_DESC_POINTER_MODE) == CUBLASLT_POINTER_MODE_DEVICE))
        return CUBLAS_STATUS_INVALID_VALUE;

    const cublasStatus_t status = dispatch(h, p, stream);  // on the call's stream; the handle's own stream is not touched
    if (status != CUBLAS_STATUS_SUCCESS || plan.gradient == 0) return status;

    // Bias gradients, as reductions that follow the product in stream order (fp32 sums in a fixed order).
    cudaError_t err = cudaSuccess;
    void* out = const_cast<void*>(biasPointer);
    if (plan.gradient == 1)  // sum over k of op(A): element (i, l) of the stored operand at i + l * lda, or l + i * lda when transposed
        err = launchVectorSums(A, la.type, ta ? la.ld : 1, ta ? 1 : la.ld, strideA, m, k, out, typeBias, biasStride, p.batch, stream);
    else if (plan.gradient == 2)  // sum over k of op(B): element (l, j) at l + j * ldb, or j + l * ldb when transposed
        err = launchVectorSums(B, lb.type, tb ? 1 : lb.ld, tb ? lb.ld : 1, strideB, n, k, out, typeBias, biasStride, p.batch, stream);
    else  // sum of the stored result over its columns (column order only: auxiliary epilogues refuse row order above)
        err = launchVectorSums(D, ld.type, 1, ld.ld, ld.batchStride, m, n, out, typeBias, biasStride, p.batch, stream);
    return err == cudaSuccess ? CUBLAS_STATUS_SUCCESS : CUBLAS_STATUS_EXECUTION_FAILED;
}

// cuBLASLt 13's grouped layouts: not served (arguments ignored).
cublasStatus_t cublasLtGroupedMatrixLayoutCreate() { return CUBLAS_STATUS_NOT_SUPPORTED; }

}  // extern "C"
#pragma GCC visibility pop
