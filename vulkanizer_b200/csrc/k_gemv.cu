// Matrix-vector kernels for GEMMs with n = 1 or m = 1 (the decode shape): y = alpha M v + beta y.
//
// Same contract as k0zi/Vulkanizer's route and shader (src/cublas/cublas.cpp:736-780, src/cublas/shaders/gemv.comp:87-146):
// M is `rows` x `len` with arbitrary row and column strides, v has stride incv, y stride incy, each of
// f32 / f16 / bf16 (int8 with int32 sums), batches by stride or by pointer arrays.
//
// The work is one pass over M, so the kernel is bound by HBM bandwidth. When rows are contiguous along
// the reduction (op(A) = A^T for n = 1) and 16-byte aligned, one warp streams one row with 128-bit loads,
// eight loads in flight per lane, fp32 partial sums per lane and a shuffle tree at the end; no shared memory,
// no block-level barrier. Any other layout takes the strided kernel (a thread per row, coalesced when the
// rows are interleaved in memory).
#include "epilogue.cuh"

namespace vkzb {
namespace {

struct GemvArgs {
    const void* M;
    const void* v;
    long long strideM, strideV;      // per batch entry, elements
    long long rowStride, colStride;  // elements
    long long incv;
    int typeM, typeV;
    int rows, len;
    int pointerArrays;
    int yIsRow;  // y^T = v^T M^T (the m = 1 case): element r of y is C(0, r)
    int batchOffset;
    EpilogueArgs epi;
};

__device__ __forceinline__ void basePointers(const GemvArgs& g, long long entry, const char*& M, const char*& v) {
    if (g.pointerArrays) {
        M = static_cast<const char*>(static_cast<const void* const*>(g.M)[entry]);
        v = static_cast<const char*>(static_cast<const void* const*>(g.v)[entry]);
    } else {
        M = static_cast<const char*>(g.M) + entry * g.strideM * dtypeSize(g.typeM);
        v = static_cast<const char*>(g.v) + entry * g.strideV * dtypeSize(g.typeV);
    }
}

template <typename Acc>
__device__ __forceinline__ void storeY(const Epilogue<Acc>& epi, int yIsRow, int r, Acc sum) {
    if (yIsRow) epi.store(0, r, sum);
    else epi.store(r, 0, sum);
}

// 8 x 16-bit values packed in a uint4, multiplied into fp32 partial sums.
template <bool BF16>
__device__ __forceinline__ float dot8(const uint4& a, const uint4& b, float acc) {
    const unsigned aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 fa, fb;
        if constexpr (BF16) {
            fa = make_float2(__uint_as_float(aw[i] << 16), __uint_as_float(aw[i] & 0xFFFF0000u));
            fb = make_float2(__uint_as_float(bw[i] << 16), __uint_as_float(bw[i] & 0xFFFF0000u));
        } else {
            fa = __half22float2(*reinterpret_cast<const __half2*>(&aw[i]));
            fb = __half22float2(*reinterpret_cast<const __half2*>(&bw[i]));
        }
        acc = fmaf(fa.x, fb.x, acc);
        acc = fmaf(fa.y, fb.y, acc);
    }
    return acc;
}

__device__ __forceinline__ uint4 streamLoad(const void* p) {
    // M is read exactly once: bypass L1 allocation so the vector stays cached
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

constexpr int kWarpsPerBlock = 8;
constexpr int kUnroll = 8;  // 16-byte loads in flight per lane: a row of 4096 halves is two trips to memory

// One warp per row; M and v both 16-bit of the same type, rows contiguous and 16-byte aligned, incv = 1.
template <bool BF16>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) gemvRowsVec16(const GemvArgs g) {
    const long long entry = (long long)blockIdx.y + g.batchOffset;
    const int row = blockIdx.x * kWarpsPerBlock + threadIdx.x / 32, lane = threadIdx.x % 32;
    if (row >= g.rows) return;
    const char *M, *v;
    basePointers(g, entry, M, v);
    const uint4* mrow = reinterpret_cast<const uint4*>(M + row * g.rowStride * 2);
    const uint4* vec = reinterpret_cast<const uint4*>(v);
    const int chunks = g.len / 8;  // 16-byte chunks; the host guarantees len % 8 == 0 handled below
    float acc[kUnroll] = {};
    int c = lane;
    for (; c + 32 * (kUnroll - 1) < chunks; c += 32 * kUnroll) {
        uint4 a[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) a[u] = streamLoad(mrow + c + 32 * u);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) acc[u] = dot8<BF16>(a[u], __ldg(vec + c + 32 * u), acc[u]);
    }
    for (; c < chunks; c += 32) acc[0] = dot8<BF16>(streamLoad(mrow + c), __ldg(vec + c), acc[0]);
    float sum = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
    // the ragged end of a row whose length is not a multiple of 8
    for (int i = chunks * 8 + lane; i < g.len; i += 32)
        sum = fmaf(loadAs<float>(M, row * g.rowStride + i, g.typeM), loadAs<float>(v, i, g.typeV), sum);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
    if (lane == 0) {
        Epilogue<float> epi;
        epi.init(g.epi, entry);
        storeY(epi, g.yIsRow, row, sum);
    }
}

// One warp per row, any types, rows contiguous (colStride = 1) but not necessarily aligned.
template <typename Acc>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) gemvRowsScalar(const GemvArgs g) {
    const long long entry = (long long)blockIdx.y + g.batchOffset;
    const int row = blockIdx.x * kWarpsPerBlock + threadIdx.x / 32, lane = threadIdx.x % 32;
    if (row >= g.rows) return;
    const char *M, *v;
    basePointers(g, entry, M, v);
    Acc sum = Acc(0);
    for (int i = lane; i < g.len; i += 32)
        sum += loadAs<Acc>(M, row * g.rowStride + i * g.colStride, g.typeM) * loadAs<Acc>(v, i * g.incv, g.typeV);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
    if (lane == 0) {
        Epilogue<Acc> epi;
        epi.init(g.epi, entry);
        storeY(epi, g.yIsRow, row, sum);
    }
}

// Rows interleaved in memory (rowStride = 1 is the coalesced case: y = A x with A column-major). A block
// covers 64 rows; its 4 thread rows split the reduction and meet in shared memory.
constexpr int kColRows = 64, kColSlices = 4;

template <typename Acc>
__global__ void __launch_bounds__(kColRows * kColSlices) gemvStrided(const GemvArgs g) {
    __shared__ Acc partial[kColSlices][kColRows];
    const long long entry = (long long)blockIdx.y + g.batchOffset;
    const int r = threadIdx.x % kColRows, slice = threadIdx.x / kColRows;
    const int row = blockIdx.x * kColRows + r;
    const char *M, *v;
    basePointers(g, entry, M, v);
    Acc sum = Acc(0);
    if (row < g.rows)
        for (int i = slice; i < g.len; i += kColSlices)
            sum += loadAs<Acc>(M, row * g.rowStride + i * g.colStride, g.typeM) * loadAs<Acc>(v, i * g.incv, g.typeV);
    partial[slice][r] = sum;
    __syncthreads();
    if (slice == 0 && row < g.rows) {
        Acc total = partial[0][r];
#pragma unroll
        for (int s = 1; s < kColSlices; ++s) total += partial[s][r];
        Epilogue<Acc> epi;
        epi.init(g.epi, entry);
        storeY(epi, g.yIsRow, row, total);
    }
}

constexpr int kMaxGridY = 65535;

template <typename Acc>
cudaError_t launchTyped(const Problem& p, GemvArgs& g, bool rowMajor) {
    for (int first = 0; first < p.batch; first += kMaxGridY) {
        g.batchOffset = first;
        const unsigned gy = unsigned(std::min(p.batch - first, kMaxGridY));
        if (rowMajor) {
            const dim3 grid((g.rows + kWarpsPerBlock - 1) / kWarpsPerBlock, gy);
            gemvRowsScalar<Acc><<<grid, kWarpsPerBlock * 32, 0, p.stream>>>(g);
        } else {
            const dim3 grid((g.rows + kColRows - 1) / kColRows, gy);
            gemvStrided<Acc><<<grid, kColRows * kColSlices, 0, p.stream>>>(g);
        }
        countLaunch();
        if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace

cudaError_t launchGemv(const Problem& p) {
    GemvArgs g{};
    g.len = p.k;
    g.pointerArrays = p.pointerArrays;
    g.epi = p.epi;
    // Roles as in cublas.cpp:745-757: n = 1 keeps A as the matrix; m = 1 computes C^T = op(B)^T op(A)^T.
    if (p.n == 1) {
        g.M = p.A, g.v = p.B, g.typeM = p.typeA, g.typeV = p.typeB;
        g.strideM = p.strideA, g.strideV = p.strideB;
        g.rows = p.m;
        g.rowStride = p.transA ? p.lda : 1, g.colStride = p.transA ? 1 : p.lda;
        g.incv = p.transB ? p.ldb : 1;
        g.yIsRow = 0;
    } else {
        g.M = p.B, g.v = p.A, g.typeM = p.typeB, g.typeV = p.typeA;
        g.strideM = p.strideB, g.strideV = p.strideA;
        g.rows = p.n;
        g.rowStride = p.transB ? 1 : p.ldb, g.colStride = p.transB ? p.ldb : 1;
        g.incv = p.transA ? 1 : p.lda;
        g.yIsRow = 1;
    }
    const bool rowMajor = g.colStride == 1;
    const auto aligned16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
    const bool vec16 = rowMajor && p.accType == kF32 && !p.pointerArrays && g.typeM == g.typeV &&
                       (g.typeM == kF16 || g.typeM == kBF16) && g.incv == 1 && g.len >= 8 && aligned16(g.M) &&
                       aligned16(g.v) && g.rowStride % 8 == 0 && g.strideM % 8 == 0 && g.strideV % 8 == 0;
    if (vec16) {
        for (int first = 0; first < p.batch; first += kMaxGridY) {
            g.batchOffset = first;
            const dim3 grid((g.rows + kWarpsPerBlock - 1) / kWarpsPerBlock, unsigned(std::min(p.batch - first, kMaxGridY)));
            if (g.typeM == kBF16) gemvRowsVec16<true><<<grid, kWarpsPerBlock * 32, 0, p.stream>>>(g);
            else gemvRowsVec16<false><<<grid, kWarpsPerBlock * 32, 0, p.stream>>>(g);
            countLaunch();
            if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    if (p.accType == kF64) return launchTyped<double>(p, g, rowMajor);
    if (p.accType == kS32) return launchTyped<int>(p, g, rowMajor);
    return launchTyped<float>(p, g, rowMajor);
}

}  // namespace vkzb
