// Triangular solves and batched LU / QR factorizations: cublasStrsm / Dtrsm (+Batched), cublasS/DgetrfBatched,
// cublasS/DgetrsBatched, cublasS/DgeqrfBatched.
//
// Same results as k0zi/Vulkanizer's shared linear-algebra kernels (src/linalg/linalg.cpp:254-375 and its shaders
// tri_solve.comp, lu_panel.comp / lu_update.comp, qr_panel.comp / householder_apply.comp, reached from
// src/cublas/cublas.cpp:1264-1431), with LAPACK's conventions: the LU pivot is the first largest |A(i, k)|, pivots are stored
// 1-based, a zero pivot records info = k + 1 once and leaves its column alone; a Householder reflector is dlarfg's
// (v(k) = 1 implied, tau = 0 for a column already zero below the diagonal).
//
// The reference walks a factorization column by column with two kernel launches per column (linalg.cpp:264-270). Here a
// whole factorization is ONE launch: the matrices these batched calls exist for (torch.linalg on batches of small matrices)
// fit a CTA's shared memory, so one CTA per matrix loads it once, runs every column step on chip with block-wide barriers in
// between, and writes it back once; a matrix too large for that is worked on in place in global memory by the same code.
// A single large triangular solve is blocked: 64-wide diagonal blocks are solved by the kernel, and everything beside them is
// updated by this repository's own GEMM (launchSgemm / launchGeneric).
#include <algorithm>

#include "gemm_problem.h"

namespace vkzb {
namespace {

constexpr int kSolveThreads = 256;
constexpr int kFactorThreads = 512;
constexpr int kMaxGridZ = 65535;
constexpr size_t kStageLimit = 200 * 1024;  // a matrix up to this size is staged in shared memory

// Matrices of a batch: an array of pointers, or one pointer and a stride in elements.
template <typename T>
struct Batch {
    const void* base;
    long long stride;
    int arrays;
    __device__ __forceinline__ T* entry(long long i) const {
        if (arrays) return static_cast<T* const*>(base)[i];
        return static_cast<T*>(const_cast<void*>(base)) + i * stride;
    }
};

// ---- triangular solve ---------------------------------------------------------------------------------------------------
//
// Solves T x = alpha b for `rhs` right-hand sides, T the order x order triangle op(A) restricted to `upper` or lower, one
// thread per right-hand side (each walks its own substitution; neighbouring threads read the same element of T, a broadcast
// from shared memory or one cached line). RIGHT: the right-hand sides are the rows of B (X op(A) = alpha B is
// op(A)^T X^T = alpha B^T), consecutive threads then touch consecutive addresses of B.
//   element (r, c) of T is A[r + c * lda], or A[c + r * lda] when `trans`
//   element i of right-hand side j is B[i + j * ldb], or B[j + i * ldb] when `right`
template <typename T>
struct TrsmArgs {
    Batch<T> A, B;
    long long lda, ldb;
    int order, rhs;
    int upper, trans, unit, right;  // `upper`, `trans` describe T as stored; the solve runs on op(T)
    T alpha;
    int batchOffset;
    int staged;  // T is copied to shared memory first
};

template <typename T>
__global__ void __launch_bounds__(kSolveThreads) trsmKernel(const TrsmArgs<T> g) {
    extern __shared__ unsigned char trsmShared[];
    T* tri = reinterpret_cast<T*>(trsmShared);
    const long long entry = (long long)blockIdx.z + g.batchOffset;
    const T* A = g.A.entry(entry);
    T* B = g.B.entry(entry);
    const int n = g.order;
    if (g.staged) {
        for (int i = threadIdx.x; i < n * n; i += blockDim.x) tri[i] = A[(i % n) + (long long)(i / n) * g.lda];
        __syncthreads();
    }
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= g.rhs) return;
    const long long strideI = g.right ? g.ldb : 1, strideJ = g.right ? 1 : g.ldb;
    T* x = B + j * strideJ;
    const auto at = [&](int r, int c) -> T {  // op(T)(r, c)
        const int sr = g.trans ? c : r, sc = g.trans ? r : c;
        return g.staged ? tri[sr + sc * n] : A[sr + (long long)sc * g.lda];
    };
    // op(T) is lower triangular when the stored triangle is lower and not transposed, or upper and transposed
    const bool lower = (g.upper != 0) == (g.trans != 0);
    if (lower) {
        for (int i = 0; i < n; ++i) {
            T s = g.alpha * x[i * strideI];
            for (int l = 0; l < i; ++l) s -= at(i, l) * x[l * strideI];
            x[i * strideI] = g.unit ? s : s / at(i, i);
        }
    } else {
        for (int i = n - 1; i >= 0; --i) {
            T s = g.alpha * x[i * strideI];
            for (int l = i + 1; l < n; ++l) s -= at(i, l) * x[l * strideI];
            x[i * strideI] = g.unit ? s : s / at(i, i);
        }
    }
}

template <typename T>
cudaError_t launchTrsmKernel(TrsmArgs<T> g, int batch, cudaStream_t stream) {
    if (g.order <= 0 || g.rhs <= 0 || batch <= 0) return cudaSuccess;
    const size_t bytes = size_t(g.order) * g.order * sizeof(T);
    g.staged = bytes <= 48 * 1024;
    for (int first = 0; first < batch; first += kMaxGridZ) {
        g.batchOffset = first;
        const dim3 grid((g.rhs + kSolveThreads - 1) / kSolveThreads, 1, std::min(batch - first, kMaxGridZ));
        trsmKernel<T><<<grid, kSolveThreads, g.staged ? bytes : 0, stream>>>(g);
        countLaunch();
        if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// B(rows, cols) *= alpha, for the blocked solve (the diagonal-block kernel then runs with alpha = 1).
template <typename T>
__global__ void scaleMatrixKernel(T* B, long long ldb, int rows, int cols, T alpha) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x, c = blockIdx.y;
    if (r < rows && c < cols) B[r + c * ldb] *= alpha;
}

// ---- LU with partial pivoting, one CTA per matrix --------------------------------------------------------------------------

template <typename T>
struct GetrfArgs {
    Batch<T> A;
    long long lda;
    int n;
    int* pivots;  // n per matrix, 1-based; null: no pivoting
    int* info;    // one per matrix
    int batchOffset;
    int staged;
};

template <typename T>
__global__ void __launch_bounds__(kFactorThreads) getrfKernel(const GetrfArgs<T> g) {
    extern __shared__ unsigned char luShared[];
    __shared__ T bestValue[kFactorThreads];
    __shared__ int bestRow[kFactorThreads];
    const long long entry = (long long)blockIdx.x + g.batchOffset;
    T* A = g.A.entry(entry);
    const int n = g.n, tid = threadIdx.x;
    T* M = A;
    long long ld = g.lda;
    if (g.staged) {
        M = reinterpret_cast<T*>(luShared);
        ld = n;
        for (int i = tid; i < n * n; i += kFactorThreads) M[i] = A[(i % n) + (long long)(i / n) * g.lda];
    }
    int firstZero = 0;
    __syncthreads();
    for (int k = 0; k < n; ++k) {
        int piv = k;
        if (g.pivots) {
            T best = T(-1);
            int row = k;
            for (int i = k + tid; i < n; i += kFactorThreads) {
                const T v = fabs(M[i + k * ld]);
                if (v > best) best = v, row = i;
            }
            bestValue[tid] = best, bestRow[tid] = row;
            __syncthreads();
            for (int s = kFactorThreads / 2; s > 0; s >>= 1) {
                if (tid < s) {
                    const T v = bestValue[tid + s];
                    const int r = bestRow[tid + s];
                    if (v > bestValue[tid] || (v == bestValue[tid] && r < bestRow[tid])) bestValue[tid] = v, bestRow[tid] = r;
                }
                __syncthreads();
            }
            piv = bestRow[0];
        }
        const T d = M[piv + k * ld];
        if (tid == 0) {
            if (g.pivots) g.pivots[entry * n + k] = piv + 1;
            if (d == T(0) && firstZero == 0) firstZero = k + 1;
        }
        __syncthreads();  // everyone has read the pivot before the swap moves it
        if (piv != k)
            for (int j = tid; j < n; j += kFactorThreads) {
                const T t = M[k + j * ld];
                M[k + j * ld] = M[piv + j * ld];
                M[piv + j * ld] = t;
            }
        __syncthreads();
        if (d != T(0)) {
            const T r = T(1) / d;
            for (int i = k + 1 + tid; i < n; i += kFactorThreads) M[i + k * ld] *= r;
        }
        __syncthreads();
        // trailing update A(i, j) -= A(i, k) A(k, j): threads run down the columns, so neighbours touch neighbouring rows
        const int rest = n - k - 1;
        for (int e = tid; e < rest * rest; e += kFactorThreads) {
            const int i = k + 1 + e % rest, j = k + 1 + e / rest;
            M[i + j * ld] -= M[i + k * ld] * M[k + j * ld];
        }
        __syncthreads();
    }
    if (g.staged)
        for (int i = tid; i < n * n; i += kFactorThreads) A[(i % n) + (long long)(i / n) * g.lda] = M[i];
    if (tid == 0 && g.info) g.info[entry] = firstZero;
}

// Rows of B exchanged as the pivots say (forward: as the factorization did; otherwise in reverse, undoing it).
template <typename T>
__global__ void applyPivotsKernel(Batch<T> B, long long ldb, int n, int nrhs, const int* pivots, int forward, int batchOffset) {
    const long long entry = (long long)blockIdx.y + batchOffset;
    T* b = B.entry(entry);
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= nrhs) return;
    const int* p = pivots + entry * n;
    for (int s = 0; s < n; ++s) {
        const int k = forward ? s : n - 1 - s, other = p[k] - 1;
        if (other != k) {
            const T t = b[k + j * ldb];
            b[k + j * ldb] = b[other + j * ldb];
            b[other + j * ldb] = t;
        }
    }
}

// ---- Householder QR, one CTA per matrix ----------------------------------------------------------------------------------

template <typename T>
struct GeqrfArgs {
    Batch<T> A;
    T* const* tau;  // one pointer per matrix
    long long lda;
    int m, n;
    int batchOffset;
    int staged;
};

template <typename T>
__global__ void __launch_bounds__(kFactorThreads) geqrfKernel(const GeqrfArgs<T> g) {
    extern __shared__ unsigned char qrShared[];
    __shared__ T partial[kFactorThreads];
    const long long entry = (long long)blockIdx.x + g.batchOffset;
    T* A = g.A.entry(entry);
    T* tau = g.tau[entry];
    const int m = g.m, n = g.n, tid = threadIdx.x, lane = tid % 32, warp = tid / 32;
    constexpr int kWarps = kFactorThreads / 32;
    T* M = A;
    long long ld = g.lda;
    if (g.staged) {
        M = reinterpret_cast<T*>(qrShared);
        ld = m;
        for (int i = tid; i < m * n; i += kFactorThreads) M[i] = A[(i % m) + (long long)(i / m) * g.lda];
    }
    __syncthreads();
    const int steps = m < n ? m : n;
    for (int k = 0; k < steps; ++k) {
        // the reflector of column k (dlarfg)
        T s = T(0);
        for (int i = k + 1 + tid; i < m; i += kFactorThreads) {
            const T x = M[i + k * ld];
            s += x * x;
        }
        partial[tid] = s;
        __syncthreads();
        for (int w = kFactorThreads / 2; w > 0; w >>= 1) {
            if (tid < w) partial[tid] += partial[tid + w];
            __syncthreads();
        }
        const T sigma = partial[0], alpha = M[k + k * ld];
        __syncthreads();  // everyone has read A(k, k) and the sum before either changes
        T tauK = T(0);
        if (sigma != T(0)) {
            const T beta = -(alpha < T(0) ? T(-1) : T(1)) * sqrt(alpha * alpha + sigma);
            const T scale = T(1) / (alpha - beta);
            for (int i = k + 1 + tid; i < m; i += kFactorThreads) M[i + k * ld] *= scale;
            tauK = (beta - alpha) / beta;
            if (tid == 0) M[k + k * ld] = beta;
        }
        if (tid == 0) tau[k] = tauK;
        __syncthreads();
        if (tauK == T(0)) continue;  // H = I
        // H applied to the trailing columns, a warp per column: w = v^T a, a -= tau w v (v(k) = 1 implied)
        for (int j = k + 1 + warp; j < n; j += kWarps) {
            T w = T(0);
            for (int i = k + 1 + lane; i < m; i += 32) w += M[i + k * ld] * M[i + j * ld];
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) w += __shfl_xor_sync(0xFFFFFFFFu, w, d);
            w += M[k + j * ld];
            __syncwarp();  // every lane has read A(k, j) before lane 0 replaces it
            const T f = tauK * w;
            if (lane == 0) M[k + j * ld] -= f;
            for (int i = k + 1 + lane; i < m; i += 32) M[i + j * ld] -= f * M[i + k * ld];
        }
        __syncthreads();
    }
    if (g.staged)
        for (int i = tid; i < m * n; i += kFactorThreads) A[(i % m) + (long long)(i / m) * g.lda] = M[i];
}

template <typename K>
cudaError_t allowSharedMemory(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return cudaSuccess;
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes));
}

// The update beside a solved diagonal block of the blocked solve: C -= op(A) op(B) through this repository's GEMM kernels.
template <typename T>
cudaError_t gemmUpdate(bool transA, bool transB, int m, int n, int k, const T* A, long long lda, const T* B, long long ldb, T* C, long long ldc,
                       cudaStream_t stream) {
    if (m <= 0 || n <= 0 || k <= 0) return cudaSuccess;
    Problem p;
    p.transA = transA, p.transB = transB;
    p.m = m, p.n = n, p.k = k, p.batch = 1;
    p.A = A, p.B = B;
    p.typeA = p.typeB = sizeof(T) == 8 ? kF64 : kF32;
    p.lda = lda, p.ldb = ldb;
    p.accType = sizeof(T) == 8 ? kF64 : kF32;
    p.epi.D = C, p.epi.C = C;
    p.epi.ldd = p.epi.ldc = ldc;
    p.epi.typeD = p.epi.typeC = p.typeA;
    p.epi.scalars.type = sizeof(T) == 8 ? kScalarF64 : kScalarF32;
    p.epi.scalars.alphaHost = -1.0, p.epi.scalars.betaHost = 1.0;
    p.stream = stream;
    return sgemmEligible(p) ? launchSgemm(p) : launchGeneric(p);
}

}  // namespace

// op(A) X = alpha B (left) or X op(A) = alpha B (right), X overwriting B; A and B as a pointer-array batch, a strided batch
// or single matrices (batch = 1).
template <typename T>
cudaError_t launchTrsm(bool right, bool upper, bool trans, bool unit, int m, int n, double alpha, const void* A, long long lda, const void* B,
                       long long ldb, int batch, bool arrays, cudaStream_t stream) {
    const int order = right ? n : m, rhs = right ? m : n;
    TrsmArgs<T> g{};
    g.A = {A, 0, arrays}, g.B = {B, 0, arrays};
    g.lda = lda, g.ldb = ldb;
    g.order = order, g.rhs = rhs;
    g.upper = upper, g.unit = unit, g.right = right;
    // X op(A) = B is op(A)^T X^T = B^T: the triangle runs transposed against what the caller asked for
    g.trans = trans != right;
    g.alpha = T(alpha);
    constexpr int kBlock = 64;
    if (arrays || batch != 1 || order <= 4 * kBlock) return launchTrsmKernel(g, batch, stream);

    // One large system: diagonal blocks of 64 by the kernel, the rest of B updated by GEMMs as each block of X is known.
    const T* a = static_cast<const T*>(A);
    T* b = static_cast<T*>(const_cast<void*>(B));
    if (alpha != 1.0) {
        scaleMatrixKernel<T><<<dim3((m + 255) / 256, n), 256, 0, stream>>>(b, ldb, m, n, T(alpha));
        countLaunch();
        if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
        g.alpha = T(1);
    }
    const bool lowerSolve = upper == g.trans;  // the order in which the unknowns fall out: first to last, or last to first
    const int blocks = (order + kBlock - 1) / kBlock;
    for (int s = 0; s < blocks; ++s) {
        const int blk = lowerSolve ? s : blocks - 1 - s, k0 = blk * kBlock, kb = std::min(kBlock, order - k0);
        TrsmArgs<T> d = g;
        d.order = kb;
        d.A = {a + k0 + (long long)k0 * lda, 0, 0};
        d.B = {right ? b + (long long)k0 * ldb : b + k0, 0, 0};
        if (cudaError_t e = launchTrsmKernel(d, 1, stream); e != cudaSuccess) return e;
        // the unknowns still to come: after this block for a forward solve, before it for a backward one
        const int r0 = lowerSolve ? k0 + kb : 0, rn = lowerSolve ? order - r0 : k0;
        if (rn <= 0) continue;
        cudaError_t e;
        if (!right) {
            // B(r, :) -= op(A)(r, k) X(k, :); op(A)(r, k) is A(r0.., k0..) or, transposed, A(k0.., r0..)^T
            const T* blockA = trans ? a + k0 + (long long)r0 * lda : a + r0 + (long long)k0 * lda;
            e = gemmUpdate<T>(trans, false, rn, n, kb, blockA, lda, b + k0, ldb, b + r0, ldb, stream);
        } else {
            // B(:, r) -= X(:, k) op(A)(k, r); op(A)(k, r) is A(k0.., r0..) or, transposed, A(r0.., k0..)^T
            const T* blockA = trans ? a + r0 + (long long)k0 * lda : a + k0 + (long long)r0 * lda;
            e = gemmUpdate<T>(false, trans, m, rn, kb, b + (long long)k0 * ldb, ldb, blockA, lda, b + (long long)r0 * ldb, ldb, stream);
        }
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

template <typename T>
cudaError_t launchGetrf(int n, const void* A, long long lda, int* pivots, int* info, int batch, cudaStream_t stream) {
    if (batch <= 0) return cudaSuccess;
    if (n == 0) return info ? cudaMemsetAsync(info, 0, size_t(batch) * sizeof(int), stream) : cudaSuccess;
    GetrfArgs<T> g{{A, 0, 1}, lda, n, pivots, info, 0, 0};
    const size_t bytes = size_t(n) * n * sizeof(T);
    g.staged = bytes <= kStageLimit;
    if (g.staged)
        if (cudaError_t e = allowSharedMemory(getrfKernel<T>, bytes); e != cudaSuccess) return e;
    for (int first = 0; first < batch; first += kMaxGridZ) {
        g.batchOffset = first;
        getrfKernel<T><<<std::min(batch - first, kMaxGridZ), kFactorThreads, g.staged ? bytes : 0, stream>>>(g);
        countLaunch();
        if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// A = P L U. A X = B: L Y = P^T B, then U X = Y. A^T X = B: U^T Y = B, L^T Z = Y, X = P Z (linalg.cpp:275-286).
template <typename T>
cudaError_t launchGetrs(bool trans, int n, int nrhs, const void* A, long long lda, const int* pivots, const void* B, long long ldb, int batch,
                        cudaStream_t stream) {
    if (n <= 0 || nrhs <= 0 || batch <= 0) return cudaSuccess;
    const auto permute = [&](bool forward) -> cudaError_t {
        if (!pivots) return cudaSuccess;
        for (int first = 0; first < batch; first += kMaxGridZ) {
            applyPivotsKernel<T><<<dim3((nrhs + 127) / 128, std::min(batch - first, kMaxGridZ)), 128, 0, stream>>>(Batch<T>{B, 0, 1}, ldb, n, nrhs, pivots,
                                                                                                                     forward, first);
            countLaunch();
            if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
        }
        return cudaSuccess;
    };
    cudaError_t e = cudaSuccess;
    if (!trans) {
        if ((e = permute(true)) != cudaSuccess) return e;
        if ((e = launchTrsm<T>(false, false, false, true, n, nrhs, 1.0, A, lda, B, ldb, batch, true, stream)) != cudaSuccess) return e;
        return launchTrsm<T>(false, true, false, false, n, nrhs, 1.0, A, lda, B, ldb, batch, true, stream);
    }
    if ((e = launchTrsm<T>(false, true, true, false, n, nrhs, 1.0, A, lda, B, ldb, batch, true, stream)) != cudaSuccess) return e;
    if ((e = launchTrsm<T>(false, false, true, true, n, nrhs, 1.0, A, lda, B, ldb, batch, true, stream)) != cudaSuccess) return e;
    return permute(false);
}

template <typename T>
cudaError_t launchGeqrf(int m, int n, const void* A, long long lda, const void* tau, int batch, cudaStream_t stream) {
    if (m <= 0 || n <= 0 || batch <= 0) return cudaSuccess;
    GeqrfArgs<T> g{{A, 0, 1}, static_cast<T* const*>(tau), lda, m, n, 0, 0};
    const size_t bytes = size_t(m) * n * sizeof(T);
    g.staged = bytes <= kStageLimit;
    if (g.staged)
        if (cudaError_t e = allowSharedMemory(geqrfKernel<T>, bytes); e != cudaSuccess) return e;
    for (int first = 0; first < batch; first += kMaxGridZ) {
        g.batchOffset = first;
        geqrfKernel<T><<<std::min(batch - first, kMaxGridZ), kFactorThreads, g.staged ? bytes : 0, stream>>>(g);
        countLaunch();
        if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

template cudaError_t launchTrsm<float>(bool, bool, bool, bool, int, int, double, const void*, long long, const void*, long long, int, bool, cudaStream_t);
template cudaError_t launchTrsm<double>(bool, bool, bool, bool, int, int, double, const void*, long long, const void*, long long, int, bool, cudaStream_t);
template cudaError_t launchGetrf<float>(int, const void*, long long, int*, int*, int, cudaStream_t);
template cudaError_t launchGetrf<double>(int, const void*, long long, int*, int*, int, cudaStream_t);
template cudaError_t launchGetrs<float>(bool, int, int, const void*, long long, const int*, const void*, long long, int, cudaStream_t);
template cudaError_t launchGetrs<double>(bool, int, int, const void*, long long, const int*, const void*, long long, int, cudaStream_t);
template cudaError_t launchGeqrf<float>(int, int, const void*, long long, const void*, int, cudaStream_t);
template cudaError_t launchGeqrf<double>(int, int, const void*, long long, const void*, int, cudaStream_t);

}  // namespace vkzb
