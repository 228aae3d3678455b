/*
 * C ABI of the B200-native libcublas.so.12 built by this repository.
 *
 * Every function below is exported with NVIDIA's documented name and signature at symbol version
 * node `libcublas.so.12`, so a program built against NVIDIA's cublas_v2.h (or against the clean-room
 * header of k0zi/Vulkanizer, include/cublas/cublas_v2.h) binds to it unchanged. This header is what
 * the repository itself compiles against; enum values follow the documented cuBLAS ABI.
 *
 * Each declaration names the Vulkanizer entry point it replaces as `src/cublas/cublas.cpp:<line>`.
 * Matrices are column-major device memory owned by the caller; sizes are `int` (the `_64` forms take
 * int64_t and refuse values beyond INT32_MAX); strides are in elements; alpha and beta have the
 * scalar type of the compute type and live on the host or on the device according to the handle's
 * pointer mode. Calls are asynchronous on the handle's stream and never synchronise it.
 */
#ifndef VKZB_CUBLAS_H
#define VKZB_CUBLAS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- types shared with the CUDA toolkit (library_types.h / driver_types.h) ---- */
#ifndef VKZB_HAVE_CUDA_TYPES
typedef struct CUstream_st* cudaStream_t;
typedef enum cudaDataType_t {
    CUDA_R_32F = 0, CUDA_R_64F = 1, CUDA_R_16F = 2, CUDA_R_8I = 3, CUDA_C_32F = 4, CUDA_C_64F = 5,
    CUDA_C_16F = 6, CUDA_C_8I = 7, CUDA_R_8U = 8, CUDA_C_8U = 9, CUDA_R_32I = 10, CUDA_C_32I = 11,
    CUDA_R_32U = 12, CUDA_C_32U = 13, CUDA_R_16BF = 14, CUDA_C_16BF = 15
} cudaDataType;
typedef enum libraryPropertyType_t { MAJOR_VERSION = 0, MINOR_VERSION = 1, PATCH_LEVEL = 2 } libraryPropertyType;
#endif

#define VKZB_CUBLAS_VER_MAJOR 12
#define VKZB_CUBLAS_VER_MINOR 9
#define VKZB_CUBLAS_VER_PATCH 0
#define VKZB_CUBLAS_VERSION (VKZB_CUBLAS_VER_MAJOR * 10000 + VKZB_CUBLAS_VER_MINOR * 100 + VKZB_CUBLAS_VER_PATCH)

typedef enum {
    CUBLAS_STATUS_SUCCESS = 0,
    CUBLAS_STATUS_NOT_INITIALIZED = 1,
    CUBLAS_STATUS_ALLOC_FAILED = 3,
    CUBLAS_STATUS_INVALID_VALUE = 7,
    CUBLAS_STATUS_ARCH_MISMATCH = 8,
    CUBLAS_STATUS_MAPPING_ERROR = 11,
    CUBLAS_STATUS_EXECUTION_FAILED = 13,
    CUBLAS_STATUS_INTERNAL_ERROR = 14,
    CUBLAS_STATUS_NOT_SUPPORTED = 15,
    CUBLAS_STATUS_LICENSE_ERROR = 16
} cublasStatus_t;

typedef enum { CUBLAS_OP_N = 0, CUBLAS_OP_T = 1, CUBLAS_OP_C = 2, CUBLAS_OP_CONJG = 3 } cublasOperation_t;
typedef enum { CUBLAS_POINTER_MODE_HOST = 0, CUBLAS_POINTER_MODE_DEVICE = 1 } cublasPointerMode_t;
typedef enum { CUBLAS_ATOMICS_NOT_ALLOWED = 0, CUBLAS_ATOMICS_ALLOWED = 1 } cublasAtomicsMode_t;
typedef enum { CUBLAS_FILL_MODE_LOWER = 0, CUBLAS_FILL_MODE_UPPER = 1, CUBLAS_FILL_MODE_FULL = 2 } cublasFillMode_t;
typedef enum { CUBLAS_DIAG_NON_UNIT = 0, CUBLAS_DIAG_UNIT = 1 } cublasDiagType_t;
typedef enum { CUBLAS_SIDE_LEFT = 0, CUBLAS_SIDE_RIGHT = 1 } cublasSideMode_t;

/* The algorithm argument is a hint: every value selects the same kernels (cublas_v2.h:107 of the reference). */
typedef int cublasGemmAlgo_t;
#define CUBLAS_GEMM_DEFAULT (-1)
#define CUBLAS_GEMM_DEFAULT_TENSOR_OP 99

typedef enum {
    CUBLAS_DEFAULT_MATH = 0,
    CUBLAS_TENSOR_OP_MATH = 1,
    CUBLAS_PEDANTIC_MATH = 2,
    CUBLAS_TF32_TENSOR_OP_MATH = 3,
    CUBLAS_MATH_DISALLOW_REDUCED_PRECISION_REDUCTION = 16
} cublasMath_t;

typedef enum {
    CUBLAS_COMPUTE_16F = 64,
    CUBLAS_COMPUTE_16F_PEDANTIC = 65,
    CUBLAS_COMPUTE_32F = 68,
    CUBLAS_COMPUTE_32F_PEDANTIC = 69,
    CUBLAS_COMPUTE_64F = 70,
    CUBLAS_COMPUTE_64F_PEDANTIC = 71,
    CUBLAS_COMPUTE_32I = 72,
    CUBLAS_COMPUTE_32I_PEDANTIC = 73,
    CUBLAS_COMPUTE_32F_FAST_16F = 74,
    CUBLAS_COMPUTE_32F_FAST_16BF = 75,
    CUBLAS_COMPUTE_32F_FAST_TF32 = 77
} cublasComputeType_t;

/* Opaque library context. A cuBLAS handle is also a valid cuBLASLt handle. */
typedef struct cublasContext* cublasHandle_t;

/* ---- handle and state (cublas.cpp:931-1060) ---- */
cublasStatus_t cublasCreate_v2(cublasHandle_t* handle);                                   /* cublas.cpp:931 */
cublasStatus_t cublasDestroy_v2(cublasHandle_t handle);                                   /* cublas.cpp:947 */
cublasStatus_t cublasGetVersion_v2(cublasHandle_t handle, int* version);                  /* cublas.cpp:954 */
cublasStatus_t cublasGetProperty(libraryPropertyType type, int* value);                   /* cublas.cpp:960 */
size_t cublasGetCudartVersion(void);                                                      /* cublas.cpp:966 */
cublasStatus_t cublasSetStream_v2(cublasHandle_t handle, cudaStream_t stream);            /* cublas.cpp:968 */
cublasStatus_t cublasGetStream_v2(cublasHandle_t handle, cudaStream_t* stream);           /* cublas.cpp:974 */
cublasStatus_t cublasSetWorkspace_v2(cublasHandle_t handle, void* workspace, size_t bytes); /* cublas.cpp:981 */
cublasStatus_t cublasSetPointerMode_v2(cublasHandle_t handle, cublasPointerMode_t mode);  /* cublas.cpp:985 */
cublasStatus_t cublasGetPointerMode_v2(cublasHandle_t handle, cublasPointerMode_t* mode); /* cublas.cpp:991 */
cublasStatus_t cublasSetSmCountTarget(cublasHandle_t handle, int smCountTarget);          /* cublas.cpp:998 */
cublasStatus_t cublasSetMathMode(cublasHandle_t handle, cublasMath_t mode);               /* cublas.cpp:1002 */
cublasStatus_t cublasGetMathMode(cublasHandle_t handle, cublasMath_t* mode);              /* cublas.cpp:1008 */
cublasStatus_t cublasSetAtomicsMode(cublasHandle_t handle, cublasAtomicsMode_t mode);     /* cublas.cpp:1015 */
cublasStatus_t cublasGetAtomicsMode(cublasHandle_t handle, cublasAtomicsMode_t* mode);    /* cublas.cpp:1021 */
const char* cublasGetStatusName(cublasStatus_t status);                                   /* cublas.cpp:1028 */
const char* cublasGetStatusString(cublasStatus_t status);                                 /* cublas.cpp:1044 */
cublasStatus_t cublasLoggerConfigure(int logIsOn, int logToStdOut, int logToStdErr, const char* logFileName); /* cublas.cpp:1060 */

/* ---- fp32 GEMM: C = alpha op(A) op(B) + beta C (cublas.cpp:1062-1085, 1168-1184, 1211) ---- */
cublasStatus_t cublasSgemm_v2(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int m, int n,
                              int k, const float* alpha, const float* A, int lda, const float* B, int ldb,
                              const float* beta, float* C, int ldc);                      /* cublas.cpp:1062 */
cublasStatus_t cublasSgemmBatched(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int m,
                                  int n, int k, const float* alpha, const float* const Aarray[], int lda,
                                  const float* const Barray[], int ldb, const float* beta, float* const Carray[],
                                  int ldc, int batchCount);                               /* cublas.cpp:1070 */
cublasStatus_t cublasSgemmStridedBatched(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb,
                                         int m, int n, int k, const float* alpha, const float* A, int lda,
                                         long long strideA, const float* B, int ldb, long long strideB,
                                         const float* beta, float* C, int ldc, long long strideC,
                                         int batchCount);                                 /* cublas.cpp:1078 */
cublasStatus_t cublasSgemm_v2_64(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int64_t m,
                                 int64_t n, int64_t k, const float* alpha, const float* A, int64_t lda,
                                 const float* B, int64_t ldb, const float* beta, float* C, int64_t ldc); /* cublas.cpp:1168 */
cublasStatus_t cublasSgemmStridedBatched_64(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb,
                                            int64_t m, int64_t n, int64_t k, const float* alpha, const float* A,
                                            int64_t lda, long long strideA, const float* B, int64_t ldb,
                                            long long strideB, const float* beta, float* C, int64_t ldc,
                                            long long strideC, int64_t batchCount);       /* cublas.cpp:1176 */
cublasStatus_t cublasSgemmEx(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int m, int n,
                             int k, const float* alpha, const void* A, cudaDataType Atype, int lda, const void* B,
                             cudaDataType Btype, int ldb, const float* beta, void* C, cudaDataType Ctype,
                             int ldc);                                                    /* cublas.cpp:1211 */

/* ---- fp64 GEMM (cublas.cpp:1087-1110, 1186-1201) ---- */
cublasStatus_t cublasDgemm_v2(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int m, int n,
                              int k, const double* alpha, const double* A, int lda, const double* B, int ldb,
                              const double* beta, double* C, int ldc);                    /* cublas.cpp:1087 */
cublasStatus_t cublasDgemmBatched(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int m,
                                  int n, int k, const double* alpha, const double* const Aarray[], int lda,
                                  const double* const Barray[], int ldb, const double* beta, double* const Carray[],
                                  int ldc, int batchCount);                               /* cublas.cpp:1095 */
cublasStatus_t cublasDgemmStridedBatched(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb,
                                         int m, int n, int k, const double* alpha, const double* A, int lda,
                                         long long strideA, const double* B, int ldb, long long strideB,
                                         const double* beta, double* C, int ldc, long long strideC,
                                         int batchCount);                                 /* cublas.cpp:1104 */
cublasStatus_t cublasDgemm_v2_64(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int64_t m,
                                 int64_t n, int64_t k, const double* alpha, const double* A, int64_t lda,
                                 const double* B, int64_t ldb, const double* beta, double* C, int64_t ldc); /* cublas.cpp:1186 */
cublasStatus_t cublasDgemmStridedBatched_64(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb,
                                            int64_t m, int64_t n, int64_t k, const double* alpha, const double* A,
                                            int64_t lda, long long strideA, const double* B, int64_t ldb,
                                            long long strideB, const double* beta, double* C, int64_t ldc,
                                            long long strideC, int64_t batchCount);       /* cublas.cpp:1194 */

/* ---- typed GEMM: fp16 / bf16 / fp32 operands with fp32 accumulation, int8 operands with int32
 *      accumulation (CUBLAS_COMPUTE_32I, alpha and beta int32; no counterpart in the reference, which
 *      answers NOT_SUPPORTED for CUDA_R_8I: cublas.cpp:178-185, 304-308) ---- */
cublasStatus_t cublasGemmEx(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int m, int n,
                            int k, const void* alpha, const void* A, cudaDataType Atype, int lda, const void* B,
                            cudaDataType Btype, int ldb, const void* beta, void* C, cudaDataType Ctype, int ldc,
                            cublasComputeType_t computeType, cublasGemmAlgo_t algo);      /* cublas.cpp:1113 */
cublasStatus_t cublasHgemm(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int m, int n,
                           int k, const void* alpha, const void* A, int lda, const void* B, int ldb, const void* beta,
                           void* C, int ldc);                                             /* cublas.cpp:1123 */
cublasStatus_t cublasGemmBatchedEx(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int m,
                                   int n, int k, const void* alpha, const void* const Aarray[], cudaDataType Atype,
                                   int lda, const void* const Barray[], cudaDataType Btype, int ldb, const void* beta,
                                   void* const Carray[], cudaDataType Ctype, int ldc, int batchCount,
                                   cublasComputeType_t computeType, cublasGemmAlgo_t algo); /* cublas.cpp:1131 */
cublasStatus_t cublasGemmStridedBatchedEx(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb,
                                          int m, int n, int k, const void* alpha, const void* A, cudaDataType Atype,
                                          int lda, long long strideA, const void* B, cudaDataType Btype, int ldb,
                                          long long strideB, const void* beta, void* C, cudaDataType Ctype, int ldc,
                                          long long strideC, int batchCount, cublasComputeType_t computeType,
                                          cublasGemmAlgo_t algo);                          /* cublas.cpp:1253 */
cublasStatus_t cublasGemmGroupedBatchedEx(cublasHandle_t handle, const cublasOperation_t transa_array[],
                                          const cublasOperation_t transb_array[], const int m_array[],
                                          const int n_array[], const int k_array[], const void* alpha_array,
                                          const void* const Aarray[], cudaDataType Atype, const int lda_array[],
                                          const void* const Barray[], cudaDataType Btype, const int ldb_array[],
                                          const void* beta_array, void* const Carray[], cudaDataType Ctype,
                                          const int ldc_array[], int group_count, const int group_size[],
                                          cublasComputeType_t computeType);               /* cublas.cpp:1221 */

/* ---- matrix-vector product, routed as an m = 1 GEMM (cublas.cpp:1143-1159, 1204) ---- */
cublasStatus_t cublasSgemv_v2(cublasHandle_t handle, cublasOperation_t trans, int m, int n, const float* alpha,
                              const float* A, int lda, const float* x, int incx, const float* beta, float* y,
                              int incy);                                                  /* cublas.cpp:1143 */
cublasStatus_t cublasSgemv_v2_64(cublasHandle_t handle, cublasOperation_t trans, int64_t m, int64_t n,
                                 const float* alpha, const float* A, int64_t lda, const float* x, int64_t incx,
                                 const float* beta, float* y, int64_t incy);              /* cublas.cpp:1204 */

/* ---- triangular solves and batched LU / QR (LAPACK conventions; csrc/k_solve.cu) ----
 * op(A) X = alpha B (left) or X op(A) = alpha B (right), X overwriting B; only the `uplo` triangle of A is read. */
cublasStatus_t cublasStrsm_v2(cublasHandle_t handle, cublasSideMode_t side, cublasFillMode_t uplo, cublasOperation_t trans,
                              cublasDiagType_t diag, int m, int n, const float* alpha, const float* A, int lda, float* B,
                              int ldb);                                                   /* cublas.cpp:1402 */
cublasStatus_t cublasDtrsm_v2(cublasHandle_t handle, cublasSideMode_t side, cublasFillMode_t uplo, cublasOperation_t trans,
                              cublasDiagType_t diag, int m, int n, const double* alpha, const double* A, int lda, double* B,
                              int ldb);                                                   /* cublas.cpp:1408 */
cublasStatus_t cublasStrsmBatched(cublasHandle_t handle, cublasSideMode_t side, cublasFillMode_t uplo, cublasOperation_t trans,
                                  cublasDiagType_t diag, int m, int n, const float* alpha, const float* const A[], int lda,
                                  float* const B[], int ldb, int batchCount);             /* cublas.cpp:1264 */
cublasStatus_t cublasDtrsmBatched(cublasHandle_t handle, cublasSideMode_t side, cublasFillMode_t uplo, cublasOperation_t trans,
                                  cublasDiagType_t diag, int m, int n, const double* alpha, const double* const A[], int lda,
                                  double* const B[], int ldb, int batchCount);            /* cublas.cpp:1414 */
/* P A = L U per matrix, in place: P receives 1-based pivot rows (n per matrix; null: no pivoting), the DEVICE array `info`
 * the first zero pivot of each matrix (0: none). */
cublasStatus_t cublasSgetrfBatched(cublasHandle_t handle, int n, float* const A[], int lda, int* P, int* info,
                                   int batchSize);                                        /* cublas.cpp:1336 */
cublasStatus_t cublasDgetrfBatched(cublasHandle_t handle, int n, double* const A[], int lda, int* P, int* info,
                                   int batchSize);                                        /* cublas.cpp:1340 */
/* op(A) X = B from the factorization above, X overwriting B. `info` is a HOST integer: 0, or minus the position of the first
 * invalid argument. */
cublasStatus_t cublasSgetrsBatched(cublasHandle_t handle, cublasOperation_t trans, int n, int nrhs, const float* const A[],
                                   int lda, const int* devIpiv, float* const B[], int ldb, int* info,
                                   int batchSize);                                        /* cublas.cpp:1344 */
cublasStatus_t cublasDgetrsBatched(cublasHandle_t handle, cublasOperation_t trans, int n, int nrhs, const double* const A[],
                                   int lda, const int* devIpiv, double* const B[], int ldb, int* info,
                                   int batchSize);                                        /* cublas.cpp:1349 */
/* A = Q R per matrix, in place as LAPACK's geqrf stores it (R on and above the diagonal, the reflectors below, their scalars
 * in tau[i][0 .. min(m, n))). `info` is a HOST integer as for getrs. */
cublasStatus_t cublasSgeqrfBatched(cublasHandle_t handle, int m, int n, float* const A[], int lda, float* const tau[],
                                   int* info, int batchSize);                             /* cublas.cpp:1420 */
cublasStatus_t cublasDgeqrfBatched(cublasHandle_t handle, int m, int n, double* const A[], int lda, double* const tau[],
                                   int* info, int batchSize);                             /* cublas.cpp:1425 */

#ifdef __cplusplus
}
#endif
#endif /* VKZB_CUBLAS_H */
