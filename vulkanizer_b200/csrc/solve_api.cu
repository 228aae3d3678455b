// libcublas.so.12 entry points for triangular solves and batched LU / QR: cublasStrsm_v2, cublasDtrsm_v2, cublasStrsmBatched,
// cublasDtrsmBatched, cublasS/DgetrfBatched, cublasS/DgetrsBatched, cublasS/DgeqrfBatched.
//
// Argument checks, status codes and the meaning of `info` follow k0zi/Vulkanizer's src/cublas/cublas.cpp:1264-1431: the
// factorizations' `info` is a device array that receives the first zero pivot of each matrix; the solvers' and QR's `info` is
// a HOST integer that reports the first invalid argument (as -position) and nothing else. alpha is read on the host, or from
// device memory with a blocking copy when the handle is in device pointer mode (a triangular solve is not a capture-critical
// path; the GEMM entry points never block).
#include <algorithm>

#define VKZB_HAVE_CUDA_TYPES
#include <library_types.h>

#include "../../include/vkzb_cublas.h"
#include "blas_internal.h"

namespace {

using namespace vkzb;

template <typename T>
bool readAlpha(cublasHandle_t h, const T* alpha, double& out) {
    if (!alpha) return false;
    if (h->pointerMode == CUBLAS_POINTER_MODE_DEVICE) {
        T v;
        if (cudaMemcpyAsync(&v, alpha, sizeof v, cudaMemcpyDeviceToHost, h->stream) != cudaSuccess || cudaStreamSynchronize(h->stream) != cudaSuccess) return false;
        out = double(v);
    } else {
        out = double(*alpha);
    }
    return true;
}

template <typename T>
cublasStatus_t trsm(cublasHandle_t h, cublasSideMode_t side, cublasFillMode_t uplo, cublasOperation_t trans, cublasDiagType_t diag, int m, int n,
                    const T* alpha, const void* A, int lda, const void* B, int ldb, int batch, bool arrays) {
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    const int order = side == CUBLAS_SIDE_LEFT ? m : n;
    if (m < 0 || n < 0 || batch < 0 || lda < std::max(1, order) || ldb < std::max(1, m) ||
        (uplo != CUBLAS_FILL_MODE_LOWER && uplo != CUBLAS_FILL_MODE_UPPER) || unsigned(trans) > CUBLAS_OP_C ||
        (side != CUBLAS_SIDE_LEFT && side != CUBLAS_SIDE_RIGHT))
        return CUBLAS_STATUS_INVALID_VALUE;
    if (m == 0 || n == 0 || batch == 0) return CUBLAS_STATUS_SUCCESS;
    double a;
    if (!readAlpha(h, alpha, a)) return CUBLAS_STATUS_INVALID_VALUE;
    const cudaError_t e = launchTrsm<T>(side == CUBLAS_SIDE_RIGHT, uplo == CUBLAS_FILL_MODE_UPPER, trans != CUBLAS_OP_N, diag == CUBLAS_DIAG_UNIT, m, n, a,
                                        A, lda, B, ldb, batch, arrays, h->stream);
    return e == cudaSuccess ? CUBLAS_STATUS_SUCCESS : CUBLAS_STATUS_EXECUTION_FAILED;
}

template <typename T>
cublasStatus_t getrf(cublasHandle_t h, int n, const void* A, int lda, int* pivots, int* info, int batch) {
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    if (n < 0 || lda < std::max(1, n) || batch < 0) return CUBLAS_STATUS_INVALID_VALUE;
    return launchGetrf<T>(n, A, lda, pivots, info, batch, h->stream) == cudaSuccess ? CUBLAS_STATUS_SUCCESS : CUBLAS_STATUS_EXECUTION_FAILED;
}

template <typename T>
cublasStatus_t getrs(cublasHandle_t h, cublasOperation_t trans, int n, int nrhs, const void* A, int lda, const int* pivots, const void* B, int ldb,
                     int* info, int batch) {
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    int bad = 0;
    if (n < 0) bad = -2;
    else if (nrhs < 0) bad = -3;
    else if (lda < std::max(1, n)) bad = -5;
    else if (ldb < std::max(1, n)) bad = -8;
    else if (batch < 0) bad = -10;
    if (info) *info = bad;
    if (bad) return CUBLAS_STATUS_INVALID_VALUE;
    return launchGetrs<T>(trans != CUBLAS_OP_N, n, nrhs, A, lda, pivots, B, ldb, batch, h->stream) == cudaSuccess ? CUBLAS_STATUS_SUCCESS
                                                                                                                 : CUBLAS_STATUS_EXECUTION_FAILED;
}

template <typename T>
cublasStatus_t geqrf(cublasHandle_t h, int m, int n, const void* A, int lda, const void* tau, int* info, int batch) {
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    int bad = 0;
    if (m < 0) bad = -1;
    else if (n < 0) bad = -2;
    else if (lda < std::max(1, m)) bad = -4;
    else if (batch < 0) bad = -7;
    if (info) *info = bad;
    if (bad) return CUBLAS_STATUS_INVALID_VALUE;
    return launchGeqrf<T>(m, n, A, lda, tau, batch, h->stream) == cudaSuccess ? CUBLAS_STATUS_SUCCESS : CUBLAS_STATUS_EXECUTION_FAILED;
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

cublasStatus_t cublasStrsm_v2(cublasHandle_t h, cublasSideMode_t side, cublasFillMode_t uplo, cublasOperation_t trans, cublasDiagType_t diag, int m,
                              int n, const float* alpha, const float* A, int lda, float* B, int ldb) {
    VKZB_API_SCOPE();
    return trsm<float>(h, side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, 1, false);
}

cublasStatus_t cublasDtrsm_v2(cublasHandle_t h, cublasSideMode_t side, cublasFillMode_t uplo, cublasOperation_t trans, cublasDiagType_t diag, int m,
                              int n, const double* alpha, const double* A, int lda, double* B, int ldb) {
    VKZB_API_SCOPE();
    return trsm<double>(h, side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, 1, false);
}

cublasStatus_t cublasStrsmBatched(cublasHandle_t h, cublasSideMode_t side, cublasFillMode_t uplo, cublasOperation_t trans, cublasDiagType_t diag, int m,
                                  int n, const float* alpha, const float* const A[], int lda, float* const B[], int ldb, int batchCount) {
    VKZB_API_SCOPE();
    return trsm<float>(h, side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, batchCount, true);
}

cublasStatus_t cublasDtrsmBatched(cublasHandle_t h, cublasSideMode_t side, cublasFillMode_t uplo, cublasOperation_t trans, cublasDiagType_t diag, int m,
                                  int n, const double* alpha, const double* const A[], int lda, double* const B[], int ldb, int batchCount) {
    VKZB_API_SCOPE();
    return trsm<double>(h, side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, batchCount, true);
}

cublasStatus_t cublasSgetrfBatched(cublasHandle_t h, int n, float* const A[], int lda, int* P, int* info, int batchSize) {
    VKZB_API_SCOPE();
    return getrf<float>(h, n, A, lda, P, info, batchSize);
}

cublasStatus_t cublasDgetrfBatched(cublasHandle_t h, int n, double* const A[], int lda, int* P, int* info, int batchSize) {
    VKZB_API_SCOPE();
    return getrf<double>(h, n, A, lda, P, info, batchSize);
}

cublasStatus_t cublasSgetrsBatched(cublasHandle_t h, cublasOperation_t trans, int n, int nrhs, const float* const A[], int lda, const int* devIpiv,
                                   float* const B[], int ldb, int* info, int batchSize) {
    VKZB_API_SCOPE();
    return getrs<float>(h, trans, n, nrhs, A, lda, devIpiv, B, ldb, info, batchSize);
}

cublasStatus_t cublasDgetrsBatched(cublasHandle_t h, cublasOperation_t trans, int n, int nrhs, const double* const A[], int lda, const int* devIpiv,
                                   double* const B[], int ldb, int* info, int batchSize) {
    VKZB_API_SCOPE();
    return getrs<double>(h, trans, n, nrhs, A, lda, devIpiv, B, ldb, info, batchSize);
}

cublasStatus_t cublasSgeqrfBatched(cublasHandle_t h, int m, int n, float* const A[], int lda, float* const tau[], int* info, int batchSize) {
    VKZB_API_SCOPE();
    return geqrf<float>(h, m, n, A, lda, tau, info, batchSize);
}

cublasStatus_t cublasDgeqrfBatched(cublasHandle_t h, int m, int n, double* const A[], int lda, double* const tau[], int* info, int batchSize) {
    VKZB_API_SCOPE();
    return geqrf<double>(h, m, n, A, lda, tau, info, batchSize);
}

}  // extern "C"
#pragma GCC visibility pop
