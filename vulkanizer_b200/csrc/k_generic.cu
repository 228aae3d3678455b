// CUDA-core tile kernel with the contract of k0zi/Vulkanizer's generic shader (src/cublas/shaders/gemm.comp:85-147):
// C = alpha op(A) op(B) + beta C for any mix of storage types, any leading dimensions, strided batches or
// device arrays of pointers. It is the correctness floor under the specialised kernels: calls whose
// operands are not 16-byte aligned, mix types, or pass pointer arrays land here. Accumulation is fp32 for
// floating-point storage, int32 for int8 and fp64 for doubles, with k ascending inside each thread.
#include "epilogue.cuh"

namespace vkzb {
namespace {

constexpr int kTile = 64;   // C tile edge per CTA
constexpr int kStep = 16;   // k slice per shared-memory fill
constexpr int kThreads = 256;

struct GenericArgs {
    const void* A;
    const void* B;
    long long lda, ldb, strideA, strideB;
    int typeA, typeB;
    int m, n, k;
    int transA, transB, pointerArrays;
    int batchOffset;
    EpilogueArgs epi;
};

template <typename Acc>
__global__ void __launch_bounds__(kThreads) genericGemmKernel(const GenericArgs g) {
    __shared__ Acc sA[kStep][kTile + 1];
    __shared__ Acc sB[kStep][kTile + 1];
    const long long entry = (long long)blockIdx.z + g.batchOffset;
    const char* A;
    const char* B;
    if (g.pointerArrays) {
        A = static_cast<const char*>(static_cast<const void* const*>(g.A)[entry]);
        B = static_cast<const char*>(static_cast<const void* const*>(g.B)[entry]);
    } else {
        A = static_cast<const char*>(g.A) + entry * g.strideA * dtypeSize(g.typeA);
        B = static_cast<const char*>(g.B) + entry * g.strideB * dtypeSize(g.typeB);
    }
    const int row0 = blockIdx.x * kTile, col0 = blockIdx.y * kTile;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    Acc acc[4][4] = {};
    for (int k0 = 0; k0 < g.k; k0 += kStep) {
        for (int i = threadIdx.x; i < kTile * kStep; i += kThreads) {
            // op(A)(row, l): consecutive threads walk the contiguous direction of the stored matrix
            const int r = g.transA ? i / kStep : i % kTile, l = g.transA ? i % kStep : i / kTile;
            const int row = row0 + r, kk = k0 + l;
            Acc v = Acc(0);
            if (row < g.m && kk < g.k)
                v = loadAs<Acc>(A, g.transA ? kk + row * g.lda : row + kk * g.lda, g.typeA);
            sA[l][r] = v;
        }
        for (int i = threadIdx.x; i < kTile * kStep; i += kThreads) {
            const int c = g.transB ? i % kTile : i / kStep, l = g.transB ? i / kTile : i % kStep;
            const int col = col0 + c, kk = k0 + l;
            Acc v = Acc(0);
            if (col < g.n && kk < g.k)
                v = loadAs<Acc>(B, g.transB ? col + kk * g.ldb : kk + col * g.ldb, g.typeB);
            sB[l][c] = v;
        }
        __syncthreads();
#pragma unroll
        for (int l = 0; l < kStep; ++l) {
            Acc a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = sA[l][tx + 16 * i], b[i] = sB[l][ty + 16 * i];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
        }
        __syncthreads();
    }
    Epilogue<Acc> epi;
    epi.init(g.epi, entry);
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = row0 + tx + 16 * i, col = col0 + ty + 16 * j;
            if (row < g.m && col < g.n) epi.store(row, col, acc[i][j]);
        }
}

// k = 0 (or alpha's product absent): D = act(beta C + bias), the "k = 0 scales C" case of the
// reference's acceptance test (tests/cublas.cpp:662).
template <typename Acc>
__global__ void scaleKernel(int m, int n, int batchOffset, const EpilogueArgs e) {
    const long long entry = (long long)blockIdx.z + batchOffset;
    Epilogue<Acc> epi;
    epi.init(e, entry);
    const int row = blockIdx.x * blockDim.x + threadIdx.x, col = blockIdx.y * blockDim.y + threadIdx.y;
    if (row < m && col < n) epi.store(row, col, Acc(0));
}

constexpr int kMaxGridZ = 65535;

}  // namespace

cudaError_t launchGeneric(const Problem& p) {
    GenericArgs g{p.A, p.B, p.lda, p.ldb, p.strideA, p.strideB, p.typeA, p.typeB, p.m, p.n, p.k,
                  p.transA, p.transB, p.pointerArrays, 0, p.epi};
    const dim3 block(kThreads);
    for (int first = 0; first < p.batch; first += kMaxGridZ) {
        g.batchOffset = first;
        const dim3 grid((p.m + kTile - 1) / kTile, (p.n + kTile - 1) / kTile, std::min(p.batch - first, kMaxGridZ));
        if (p.accType == kF64) genericGemmKernel<double><<<grid, block, 0, p.stream>>>(g);
        else if (p.accType == kS32) genericGemmKernel<int><<<grid, block, 0, p.stream>>>(g);
        else genericGemmKernel<float><<<grid, block, 0, p.stream>>>(g);
        countLaunch();
        if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

cudaError_t launchScale(const Problem& p) {
    const dim3 block(64, 4);
    for (int first = 0; first < p.batch; first += kMaxGridZ) {
        const dim3 grid((p.m + 63) / 64, (p.n + 3) / 4, std::min(p.batch - first, kMaxGridZ));
        if (p.accType == kF64) scaleKernel<double><<<grid, block, 0, p.stream>>>(p.m, p.n, first, p.epi);
        else if (p.accType == kS32) scaleKernel<int><<<grid, block, 0, p.stream>>>(p.m, p.n, first, p.epi);
        else scaleKernel<float><<<grid, block, 0, p.stream>>>(p.m, p.n, first, p.epi);
        countLaunch();
        if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace vkzb
