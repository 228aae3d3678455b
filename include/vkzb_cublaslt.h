/*
 * C ABI of the B200-native libcublasLt.so.12 built by this repository (symbol version node
 * `libcublasLt.so.12`). Names, signatures and enum values are NVIDIA's documented cuBLASLt ones, so
 * programs built against NVIDIA's cublasLt.h bind unchanged. Each declaration names the Vulkanizer
 * entry point it replaces as `src/cublas/cublasLt.cpp:<line>`.
 *
 * cublasLtMatmul computes D = act(alpha op(A) op(B) + beta C + bias) in ONE kernel: bias, ReLU and
 * tanh-GELU run in the GEMM's epilogue (the reference runs a second pass over D, cublasLt.cpp:386-412),
 * and C is read in place of D when C != D (the reference copies C into D first, cublasLt.cpp:363-378).
 * C is never written. Supported: f32/f16/bf16 matrices with f32 accumulation, int8 operands with int32
 * C/D (default epilogue), transc = N, column or row order per matrix (C and D in the same order).
 * Epilogues: DEFAULT, RELU, BIAS, RELU_BIAS, GELU, GELU_BIAS as in the reference, and beyond it
 * (the reference answers NOT_SUPPORTED, cublasLt.cpp:68-78) NVIDIA's auxiliary and backward forms,
 * for D in column order:
 *   RELU_AUX(_BIAS)   also writes a bit mask: bit (row + col * aux_ld) of the auxiliary matrix is 1 where
 *                     the value before ReLU was > 0 (aux_ld counts bits, a multiple of 32, >= rows)
 *   GELU_AUX(_BIAS)   also writes the value before GELU to the auxiliary matrix (aux_ld >= rows)
 *   DRELU, DGELU      D = (alpha op(A) op(B) + beta C) * activation'(forward input), the mask or input
 *                     matrix of the forward pass being read from the auxiliary pointer
 *   DRELU_BGRAD, DGELU_BGRAD   the same, then bias[i] = sum over columns of D(i, :) (fp32 sums of the
 *                     stored D, fixed order), written to the bias pointer
 *   BGRADA, BGRADB    the plain product, and bias[i] = sum over k of op(A)(i, :) (length m), or
 *                     bias[j] = sum over k of op(B)(:, j) (length n)
 * Anything else answers CUBLAS_STATUS_NOT_SUPPORTED from the heuristic, the check and the matmul alike.
 */
#ifndef VKZB_CUBLASLT_H
#define VKZB_CUBLASLT_H

#include "vkzb_cublas.h"

#ifdef __cplusplus
extern "C" {
#endif

/* A cuBLAS handle is accepted wherever a cuBLASLt handle is (cublasLt.cpp:137-138). */
typedef struct cublasContext* cublasLtHandle_t;
typedef struct cublasLtMatmulDescOpaque_st* cublasLtMatmulDesc_t;
typedef struct cublasLtMatrixLayoutOpaque_st* cublasLtMatrixLayout_t;
typedef struct cublasLtMatmulPreferenceOpaque_st* cublasLtMatmulPreference_t;

typedef struct { uint64_t data[8]; } cublasLtMatmulAlgo_t;
typedef struct {
    cublasLtMatmulAlgo_t algo;
    size_t workspaceSize;
    cublasStatus_t state;
    float wavesCount;
    int reserved[4];
} cublasLtMatmulHeuristicResult_t;

typedef enum { CUBLASLT_ORDER_COL = 0, CUBLASLT_ORDER_ROW = 1 } cublasLtOrder_t;
typedef enum { CUBLASLT_POINTER_MODE_HOST = 0, CUBLASLT_POINTER_MODE_DEVICE = 1 } cublasLtPointerMode_t;

typedef enum {
    CUBLASLT_MATRIX_LAYOUT_TYPE = 0,
    CUBLASLT_MATRIX_LAYOUT_ORDER = 1,
    CUBLASLT_MATRIX_LAYOUT_ROWS = 2,
    CUBLASLT_MATRIX_LAYOUT_COLS = 3,
    CUBLASLT_MATRIX_LAYOUT_LD = 4,
    CUBLASLT_MATRIX_LAYOUT_BATCH_COUNT = 5,
    CUBLASLT_MATRIX_LAYOUT_STRIDED_BATCH_OFFSET = 6
} cublasLtMatrixLayoutAttribute_t;

typedef enum {
    CUBLASLT_MATMUL_DESC_COMPUTE_TYPE = 0,
    CUBLASLT_MATMUL_DESC_SCALE_TYPE = 1,
    CUBLASLT_MATMUL_DESC_POINTER_MODE = 2,
    CUBLASLT_MATMUL_DESC_TRANSA = 3,
    CUBLASLT_MATMUL_DESC_TRANSB = 4,
    CUBLASLT_MATMUL_DESC_TRANSC = 5,
    CUBLASLT_MATMUL_DESC_FILL_MODE = 6,
    CUBLASLT_MATMUL_DESC_EPILOGUE = 7,
    CUBLASLT_MATMUL_DESC_BIAS_POINTER = 8,
    CUBLASLT_MATMUL_DESC_BIAS_BATCH_STRIDE = 10,
    CUBLASLT_MATMUL_DESC_EPILOGUE_AUX_POINTER = 11,
    CUBLASLT_MATMUL_DESC_EPILOGUE_AUX_LD = 12,
    CUBLASLT_MATMUL_DESC_EPILOGUE_AUX_BATCH_STRIDE = 13,
    CUBLASLT_MATMUL_DESC_SM_COUNT_TARGET = 15,
    CUBLASLT_MATMUL_DESC_EPILOGUE_AUX_DATA_TYPE = 22,
    CUBLASLT_MATMUL_DESC_FAST_ACCUM = 25,
    CUBLASLT_MATMUL_DESC_BIAS_DATA_TYPE = 26
} cublasLtMatmulDescAttributes_t;

typedef enum {
    CUBLASLT_EPILOGUE_DEFAULT = 1,
    CUBLASLT_EPILOGUE_RELU = 2,
    CUBLASLT_EPILOGUE_BIAS = 4,
    CUBLASLT_EPILOGUE_RELU_BIAS = 6,
    CUBLASLT_EPILOGUE_GELU = 32,
    CUBLASLT_EPILOGUE_GELU_BIAS = 36,
    CUBLASLT_EPILOGUE_RELU_AUX = 130,
    CUBLASLT_EPILOGUE_RELU_AUX_BIAS = 134,
    CUBLASLT_EPILOGUE_DRELU = 136,
    CUBLASLT_EPILOGUE_DRELU_BGRAD = 152,
    CUBLASLT_EPILOGUE_GELU_AUX = 160,
    CUBLASLT_EPILOGUE_GELU_AUX_BIAS = 164,
    CUBLASLT_EPILOGUE_DGELU = 192,
    CUBLASLT_EPILOGUE_DGELU_BGRAD = 208,
    CUBLASLT_EPILOGUE_BGRADA = 256,
    CUBLASLT_EPILOGUE_BGRADB = 512
} cublasLtEpilogue_t;

typedef enum {
    CUBLASLT_MATMUL_PREF_SEARCH_MODE = 0,
    CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES = 1
} cublasLtMatmulPreferenceAttributes_t;

cublasStatus_t cublasLtCreate(cublasLtHandle_t* lightHandle);                              /* cublasLt.cpp:137 */
cublasStatus_t cublasLtDestroy(cublasLtHandle_t lightHandle);                              /* cublasLt.cpp:138 */
size_t cublasLtGetVersion(void);                                                           /* cublasLt.cpp:139 */
size_t cublasLtGetCudartVersion(void);                                                     /* cublasLt.cpp:140 */

cublasStatus_t cublasLtMatmulDescCreate(cublasLtMatmulDesc_t* matmulDesc, cublasComputeType_t computeType,
                                        cudaDataType scaleType);                           /* cublasLt.cpp:142 */
cublasStatus_t cublasLtMatmulDescDestroy(cublasLtMatmulDesc_t matmulDesc);                 /* cublasLt.cpp:152 */
cublasStatus_t cublasLtMatmulDescSetAttribute(cublasLtMatmulDesc_t matmulDesc, cublasLtMatmulDescAttributes_t attr,
                                              const void* buf, size_t sizeInBytes);        /* cublasLt.cpp:157 */
cublasStatus_t cublasLtMatmulDescGetAttribute(cublasLtMatmulDesc_t matmulDesc, cublasLtMatmulDescAttributes_t attr,
                                              void* buf, size_t sizeInBytes, size_t* sizeWritten); /* cublasLt.cpp:182 */

cublasStatus_t cublasLtMatrixLayoutCreate(cublasLtMatrixLayout_t* matLayout, cudaDataType type, uint64_t rows,
                                          uint64_t cols, int64_t ld);                      /* cublasLt.cpp:201 */
cublasStatus_t cublasLtMatrixLayoutDestroy(cublasLtMatrixLayout_t matLayout);              /* cublasLt.cpp:213 */
cublasStatus_t cublasLtMatrixLayoutSetAttribute(cublasLtMatrixLayout_t matLayout, cublasLtMatrixLayoutAttribute_t attr,
                                                const void* buf, size_t sizeInBytes);      /* cublasLt.cpp:218 */
cublasStatus_t cublasLtMatrixLayoutGetAttribute(cublasLtMatrixLayout_t matLayout, cublasLtMatrixLayoutAttribute_t attr,
                                                void* buf, size_t sizeInBytes, size_t* sizeWritten); /* cublasLt.cpp:236 */

cublasStatus_t cublasLtMatmulPreferenceCreate(cublasLtMatmulPreference_t* pref);           /* cublasLt.cpp:252 */
cublasStatus_t cublasLtMatmulPreferenceDestroy(cublasLtMatmulPreference_t pref);           /* cublasLt.cpp:258 */
cublasStatus_t cublasLtMatmulPreferenceSetAttribute(cublasLtMatmulPreference_t pref,
                                                    cublasLtMatmulPreferenceAttributes_t attr, const void* buf,
                                                    size_t sizeInBytes);                   /* cublasLt.cpp:263 */
cublasStatus_t cublasLtMatmulPreferenceGetAttribute(cublasLtMatmulPreference_t pref,
                                                    cublasLtMatmulPreferenceAttributes_t attr, void* buf,
                                                    size_t sizeInBytes, size_t* sizeWritten); /* cublasLt.cpp:271 */

/* One algorithm, needing no workspace, for every supported problem. */
cublasStatus_t cublasLtMatmulAlgoGetHeuristic(cublasLtHandle_t lightHandle, cublasLtMatmulDesc_t operationDesc,
                                              cublasLtMatrixLayout_t Adesc, cublasLtMatrixLayout_t Bdesc,
                                              cublasLtMatrixLayout_t Cdesc, cublasLtMatrixLayout_t Ddesc,
                                              cublasLtMatmulPreference_t preference, int requestedAlgoCount,
                                              cublasLtMatmulHeuristicResult_t heuristicResultsArray[],
                                              int* returnAlgoCount);                       /* cublasLt.cpp:280 */
cublasStatus_t cublasLtMatmulAlgoInit(cublasLtHandle_t lightHandle, cublasComputeType_t computeType,
                                      cudaDataType scaleType, cudaDataType Atype, cudaDataType Btype,
                                      cudaDataType Ctype, cudaDataType Dtype, int algoId,
                                      cublasLtMatmulAlgo_t* algo);                         /* cublasLt.cpp:299 */
cublasStatus_t cublasLtMatmulAlgoCheck(cublasLtHandle_t lightHandle, cublasLtMatmulDesc_t operationDesc,
                                       cublasLtMatrixLayout_t Adesc, cublasLtMatrixLayout_t Bdesc,
                                       cublasLtMatrixLayout_t Cdesc, cublasLtMatrixLayout_t Ddesc,
                                       const cublasLtMatmulAlgo_t* algo,
                                       cublasLtMatmulHeuristicResult_t* result);           /* cublasLt.cpp:306 */
cublasStatus_t cublasLtMatmulAlgoConfigSetAttribute(cublasLtMatmulAlgo_t* algo, int attr, const void* buf,
                                                    size_t sizeInBytes);                   /* cublasLt.cpp:320 */
cublasStatus_t cublasLtMatmulAlgoConfigGetAttribute(const cublasLtMatmulAlgo_t* algo, int attr, void* buf,
                                                    size_t sizeInBytes, size_t* sizeWritten); /* cublasLt.cpp:324 */

/* Asynchronous on `stream`. `algo`, `workspace` and `workspaceSizeInBytes` are accepted and unused. */
cublasStatus_t cublasLtMatmul(cublasLtHandle_t lightHandle, cublasLtMatmulDesc_t computeDesc, const void* alpha,
                              const void* A, cublasLtMatrixLayout_t Adesc, const void* B, cublasLtMatrixLayout_t Bdesc,
                              const void* beta, const void* C, cublasLtMatrixLayout_t Cdesc, void* D,
                              cublasLtMatrixLayout_t Ddesc, const cublasLtMatmulAlgo_t* algo, void* workspace,
                              size_t workspaceSizeInBytes, cudaStream_t stream);           /* cublasLt.cpp:333 */

#ifdef __cplusplus
}
#endif
#endif /* VKZB_CUBLASLT_H */
