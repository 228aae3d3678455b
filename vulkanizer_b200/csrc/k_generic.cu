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
    int colTileBase;  // first tile column of this launch (gridDim.y holds at most 65535 of them)
    EpilogueArgs epi;
};

// One 64 x 64 tile of one batch entry.
template <typename Acc>
__device__ __forceinline__ void genericTile(const GenericArgs& g, int tileRow, int tileCol, long long entry, Acc (&sA)[kStep][kTile + 1],
                                            Acc (&sB)[kStep][kTile + 1]) {
    const char* A;
    const char* B;
    if (g.pointerArrays) {
        A = static_cast<const char*>(static_cast<const void* const*>(g.A)[entry]);
        B = static_cast<const char*>(static_cast<const void* const*>(g.B)[entry]);
    } else {
        A = static_cast<const char*>(g.A) + entry * g.strideA * dtypeSize(g.typeA);
        B = static_cast<const char*>(g.B) + entry * g.strideB * dtypeSize(g.typeB);
    }
    const int row0 = tileRow * kTile, col0 = tileCol * kTile;
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

template <typename Acc>
__global__ void __launch_bounds__(kThreads) genericGemmKernel(const GenericArgs g) {
    __shared__ Acc sA[kStep][kTile + 1];
    __shared__ Acc sB[kStep][kTile + 1];
    genericTile<Acc>(g, blockIdx.x, blockIdx.y + g.colTileBase, (long long)blockIdx.z + g.batchOffset, sA, sB);
}

// The same as a stand-in queued behind a tensor-core launch that may have stood down (a pointer-array batch with an address
// TMA cannot take): a few blocks per SM that leave at once unless *runIfSet says the work is theirs, and then walk all the
// tiles. (A full grid of blocks that only look and leave would cost more than the tensor-core launch itself.)
template <typename Acc>
__global__ void __launch_bounds__(kThreads) genericGemmStandIn(const GenericArgs g, const unsigned* runIfEquals, unsigned value, int entries) {
    __shared__ Acc sA[kStep][kTile + 1];
    __shared__ Acc sB[kStep][kTile + 1];
    if (*runIfEquals != value) return;
    const long long tilesM = (g.m + kTile - 1) / kTile, tilesN = (g.n + kTile - 1) / kTile, total = tilesM * tilesN * entries;
    for (long long t = blockIdx.x; t < total; t += gridDim.x)
        genericTile<Acc>(g, int(t % tilesM), int(t / tilesM % tilesN), t / (tilesM * tilesN), sA, sB);
}

// k = 0 (or alpha's product absent): D = act(beta C + bias), the "k = 0 scales C" case of the
// reference's acceptance test (tests/cublas.cpp:662).
template <typename Acc>
__global__ void scaleKernel(int m, int n, int batchOffset, int colBase, const EpilogueArgs e) {
    const long long entry = (long long)blockIdx.z + batchOffset;
    Epilogue<Acc> epi;
    epi.init(e, entry);
    const int row = blockIdx.x * blockDim.x + threadIdx.x, col = colBase + blockIdx.y * blockDim.y + threadIdx.y;
    if (row < m && col < n) epi.store(row, col, Acc(0));
}

constexpr int kMaxGridZ = 65535, kMaxGridY = 65535;

// out[i] = sum over j of M(i, j), i < count, j < length, where M(i, j) lives at M[i * strideI + j * strideJ]: the bias
// gradients of the cuBLASLt epilogues (a sum of op(A) or op(B) over k, or of the result over its columns). fp32 sums in a
// fixed order, so the result is the same from run to run. ALONG_I: consecutive i are adjacent in memory, one thread per sum
// (its loads coalesce with its neighbours'); otherwise one warp per sum, lanes striding j, then a shuffle tree.
template <bool ALONG_I>
__global__ void vectorSumKernel(const void* M, int type, long long strideI, long long strideJ, long long batchStrideM, int count, int length,
                                void* out, int typeOut, long long batchStrideOut) {
    const char* src = static_cast<const char*>(M) + (long long)blockIdx.y * batchStrideM * dtypeSize(type);
    char* dst = static_cast<char*>(out) + (long long)blockIdx.y * batchStrideOut * dtypeSize(typeOut);
    if constexpr (ALONG_I) {
        const int i = blockIdx.x * blockDim.x + threadIdx.x;
        if (i >= count) return;
        float sum = 0.0f;
        for (int j = 0; j < length; ++j) sum += loadAs<float>(src, i * strideI + j * strideJ, type);
        storeFloat(dst, i, typeOut, sum);
    } else {
        const int i = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32, lane = threadIdx.x % 32;
        if (i >= count) return;
        float sum = 0.0f;
        for (int j = lane; j < length; j += 32) sum += loadAs<float>(src, i * strideI + j * strideJ, type);
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
        if (lane == 0) storeFloat(dst, i, typeOut, sum);
    }
}

}  // namespace

cudaError_t launchVectorSums(const void* M, int type, long long strideI, long long strideJ, long long batchStrideM, int count, int length,
                             void* out, int typeOut, long long batchStrideOut, int batch, cudaStream_t stream) {
    if (count <= 0 || batch <= 0) return cudaSuccess;
    for (int first = 0; first < batch; first += kMaxGridY) {
        const unsigned entries = unsigned(std::min(batch - first, kMaxGridY));
        const char* src = static_cast<const char*>(M) + (long long)first * batchStrideM * dtypeSize(type);
        char* dst = static_cast<char*>(out) + (long long)first * batchStrideOut * dtypeSize(typeOut);
        if (strideI == 1) vectorSumKernel<true><<<dim3((count + 127) / 128, entries), 128, 0, stream>>>(src, type, strideI, strideJ, batchStrideM, count, length, dst, typeOut, batchStrideOut);
        else vectorSumKernel<false><<<dim3((count + 7) / 8, entries), 256, 0, stream>>>(src, type, strideI, strideJ, batchStrideM, count, length, dst, typeOut, batchStrideOut);
        countLaunch();
        if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

cudaError_t launchGeneric(const Problem& p) {
    GenericArgs g{p.A, p.B, p.lda, p.ldb, p.strideA, p.strideB, p.typeA, p.typeB, p.m, p.n, p.k,
                  p.transA, p.transB, p.pointerArrays, 0, 0, p.epi};
    const dim3 block(kThreads);
    const int tilesN = (p.n + kTile - 1) / kTile;
    for (int first = 0; first < p.batch; first += kMaxGridZ)
        for (int tile = 0; tile < tilesN; tile += kMaxGridY) {
            g.batchOffset = first, g.colTileBase = tile;
            const dim3 grid((p.m + kTile - 1) / kTile, std::min(tilesN - tile, kMaxGridY), std::min(p.batch - first, kMaxGridZ));
            if (p.accType == kF64) genericGemmKernel<double><<<grid, block, 0, p.stream>>>(g);
            else if (p.accType == kS32) genericGemmKernel<int><<<grid, block, 0, p.stream>>>(g);
            else genericGemmKernel<float><<<grid, block, 0, p.stream>>>(g);
            countLaunch();
            if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
        }
    return cudaSuccess;
}

cudaError_t launchGenericStandIn(const Problem& p, const unsigned* runIfEquals, unsigned value) {
    GenericArgs g{p.A, p.B, p.lda, p.ldb, p.strideA, p.strideB, p.typeA, p.typeB, p.m, p.n, p.k,
                  p.transA, p.transB, p.pointerArrays, 0, 0, p.epi};
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const long long tiles = (long long)((p.m + kTile - 1) / kTile) * ((p.n + kTile - 1) / kTile) * p.batch;
    const unsigned grid = unsigned(std::min<long long>(tiles, 4LL * sms));
    if (p.accType == kS32) genericGemmStandIn<int><<<grid, kThreads, 0, p.stream>>>(g, runIfEquals, value, p.batch);
    else genericGemmStandIn<float><<<grid, kThreads, 0, p.stream>>>(g, runIfEquals, value, p.batch);
    countLaunch();
    return cudaGetLastError();
}

cudaError_t launchScale(const Problem& p) {
    const dim3 block(64, 4);
    const int groupsN = (p.n + 3) / 4;  // column groups of 4; a launch takes at most 65535 of them
    for (int first = 0; first < p.batch; first += kMaxGridZ)
        for (int group = 0; group < groupsN; group += kMaxGridY) {
            const dim3 grid((p.m + 63) / 64, std::min(groupsN - group, kMaxGridY), std::min(p.batch - first, kMaxGridZ));
            if (p.accType == kF64) scaleKernel<double><<<grid, block, 0, p.stream>>>(p.m, p.n, first, group * 4, p.epi);
            else if (p.accType == kS32) scaleKernel<int><<<grid, block, 0, p.stream>>>(p.m, p.n, first, group * 4, p.epi);
            else scaleKernel<float><<<grid, block, 0, p.stream>>>(p.m, p.n, first, group * 4, p.epi);
            countLaunch();
            if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
        }
    return cudaSuccess;
}

}  // namespace vkzb
