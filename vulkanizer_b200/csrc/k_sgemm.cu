// fp32 GEMM on the CUDA cores: register-blocked FFMA with float4-vectorised, coalesced global loads.
//
// Replaces k0zi/Vulkanizer's 128 x 128 tiled shader for fp32 operands (src/cublas/shaders/gemm_tiled.comp:178-240,
// selected at src/cublas/cublas.cpp:825-837): every transpose combination, 16-byte loads where pointer, leading
// dimension and tile offset allow, scalar loads at the ragged edges. A tile of op(A) and of op(B) is staged in
// shared memory k-major ([k][m] and [k][n]) so the inner product reads two float4 of each per k; the next k slice
// is fetched into registers while the current one is multiplied (two shared buffers, one barrier per slice).
// Accumulation is plain fp32 with k ascending, so results stay within 1e-5 of an fp64 reference.
#include <cstdio>
#include <cstdlib>

#include "epilogue.cuh"
#include "measure.h"

namespace vkzb {
namespace {

constexpr int kThreads = 256;

struct SgemmArgs {
    const float* A;
    const float* B;
    long long lda, ldb, strideA, strideB;
    int m, n, k;
    int batchOffset;
    int colTileBase;  // first tile column of this launch (gridDim.y holds at most 65535)
    EpilogueArgs epi;
    // split-k (one batch entry only): blockIdx.z is the slice of k, kPer its length; partial tiles and per-tile arrival
    // counters live in scratch memory
    int splits, kPer;
    float* partials;
    unsigned* counters;
};

// Fetches this thread's part of a BMN x BK tile of an operand into registers.
//   MN_CONTIG: element (mn, l) lives at src[mn + l * ld] (op = N for A, op = T for B)
//   else:      element (mn, l) lives at src[l + mn * ld]
template <int BMN, int BK, bool MN_CONTIG>
struct TileLoader {
    static constexpr int kVecs = BMN * BK / 4 / kThreads;  // float4 per thread
    static_assert(kVecs >= 1, "tile too small for 256 threads");
    float4 reg[kVecs];

    __device__ __forceinline__ void fetch(const float* src, long long ld, int mn0, int mnEnd, int k0, int kEnd, bool vecOk) {
#pragma unroll
        for (int v = 0; v < kVecs; ++v) {
            const int idx = threadIdx.x + v * kThreads;
            float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
            if constexpr (MN_CONTIG) {
                const int l = idx / (BMN / 4), mn = mn0 + (idx % (BMN / 4)) * 4, kk = k0 + l;
                if (kk < kEnd) {
                    const float* p = src + mn + kk * ld;
                    if (vecOk && mn + 3 < mnEnd) r = *reinterpret_cast<const float4*>(p);
                    else {
                        if (mn < mnEnd) r.x = p[0];
                        if (mn + 1 < mnEnd) r.y = p[1];
                        if (mn + 2 < mnEnd) r.z = p[2];
                        if (mn + 3 < mnEnd) r.w = p[3];
                    }
                }
            } else {
                const int mn = mn0 + idx / (BK / 4), kk = k0 + (idx % (BK / 4)) * 4;
                if (mn < mnEnd) {
                    const float* p = src + kk + mn * ld;
                    if (vecOk && kk + 3 < kEnd) r = *reinterpret_cast<const float4*>(p);
                    else {
                        if (kk < kEnd) r.x = p[0];
                        if (kk + 1 < kEnd) r.y = p[1];
                        if (kk + 2 < kEnd) r.z = p[2];
                        if (kk + 3 < kEnd) r.w = p[3];
                    }
                }
            }
            reg[v] = r;
        }
    }

    // Shared layout: tile[l][mn], row pitch BMN + 4 floats (keeps the transposing stores conflict-free).
    __device__ __forceinline__ void commit(float* tile) const {
        constexpr int kPitch = BMN + 4;
#pragma unroll
        for (int v = 0; v < kVecs; ++v) {
            const int idx = threadIdx.x + v * kThreads;
            if constexpr (MN_CONTIG) {
                const int l = idx / (BMN / 4), mn = (idx % (BMN / 4)) * 4;
                *reinterpret_cast<float4*>(tile + l * kPitch + mn) = reg[v];
            } else {
                const int mn = idx / (BK / 4), l = (idx % (BK / 4)) * 4;
                tile[(l + 0) * kPitch + mn] = reg[v].x;
                tile[(l + 1) * kPitch + mn] = reg[v].y;
                tile[(l + 2) * kPitch + mn] = reg[v].z;
                tile[(l + 3) * kPitch + mn] = reg[v].w;
            }
        }
    }
};

// BM x BN tile per CTA, (BM/16) x (BN/16) results per thread as 4-wide groups 64 (or 32) apart.
// SPLITK: the k range is cut into g.splits slices, one CTA each, for products too small to fill the SMs otherwise (512^3 is
// 64 tiles of 64 x 64 for 148 SMs, and each would walk all of k alone). A CTA leaves its partial tile in scratch memory and
// counts itself in; the last one to arrive for a tile adds the partial tiles in slice order, so the result does not depend
// on which CTA came last, applies alpha and beta, and resets the counter for the next call.
template <int BM, int BN, bool A_MCONTIG, bool B_NCONTIG, bool SPLITK = false>
__global__ void __launch_bounds__(kThreads, 2) sgemmKernel(const SgemmArgs g) {
    constexpr int TM = BM / 16, TN = BN / 16;        // 8 x 8 for 128 x 128, 4 x 4 for 64 x 64
    constexpr int GM = TM / 4, GN = TN / 4;          // float4 groups per thread
    constexpr int BK = 16;                           // k slice per shared-memory fill
    constexpr int kPitchA = BM + 4, kPitchB = BN + 4;
    __shared__ __align__(16) float sA[2][BK * kPitchA];
    __shared__ __align__(16) float sB[2][BK * kPitchB];

    const long long entry = SPLITK ? 0 : (long long)blockIdx.z + g.batchOffset;
    const float* A = g.A + entry * g.strideA;
    const float* B = g.B + entry * g.strideB;
    const int row0 = blockIdx.x * BM, col0 = (blockIdx.y + g.colTileBase) * BN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int kBegin = SPLITK ? int(blockIdx.z) * g.kPer : 0;
    const int kEnd = SPLITK ? min(g.k, kBegin + g.kPer) : g.k;

    const bool vecA = (reinterpret_cast<uintptr_t>(A) & 15) == 0 && g.lda % 4 == 0;
    const bool vecB = (reinterpret_cast<uintptr_t>(B) & 15) == 0 && g.ldb % 4 == 0;

    TileLoader<BM, BK, A_MCONTIG> la;
    TileLoader<BN, BK, B_NCONTIG> lb;
    float acc[TM][TN] = {};

    la.fetch(A, g.lda, row0, g.m, kBegin, kEnd, vecA);
    lb.fetch(B, g.ldb, col0, g.n, kBegin, kEnd, vecB);
    la.commit(sA[0]);
    lb.commit(sB[0]);
    __syncthreads();

    // The small-tile variant sums in two levels: products are added into `part` for kFlush k slices, then `part` is
    // added into `acc`. Against one long chain this halves the rounding error of a 512-term sum (the running sum that
    // each addition rounds stays small), which keeps fp32 results within 1e-5 of an fp64 reference at K = 512.
    constexpr bool kTwoLevel = BM < 128;
    constexpr int kFlush = 4;
    float part[kTwoLevel ? TM : 1][kTwoLevel ? TN : 1] = {};
    int buf = 0, sinceFlush = 0;
    for (int k0 = kBegin; k0 < kEnd; k0 += BK) {
        const bool more = k0 + BK < kEnd;
        if (more) {
            la.fetch(A, g.lda, row0, g.m, k0 + BK, kEnd, vecA);
            lb.fetch(B, g.ldb, col0, g.n, k0 + BK, kEnd, vecB);
        }
        const float* a = sA[buf];
        const float* b = sB[buf];
#pragma unroll
        for (int l = 0; l < BK; ++l) {
            float av[TM], bv[TN];
#pragma unroll
            for (int i = 0; i < GM; ++i)
                *reinterpret_cast<float4*>(&av[4 * i]) = *reinterpret_cast<const float4*>(a + l * kPitchA + tx * 4 + i * 64);
#pragma unroll
            for (int j = 0; j < GN; ++j)
                *reinterpret_cast<float4*>(&bv[4 * j]) = *reinterpret_cast<const float4*>(b + l * kPitchB + ty * 4 + j * 64);
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    if constexpr (kTwoLevel) part[i][j] = fmaf(av[i], bv[j], part[i][j]);
                    else acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
                }
        }
        if constexpr (kTwoLevel) {
            if (++sinceFlush == kFlush || !more) {
                sinceFlush = 0;
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) acc[i][j] += part[i][j], part[i][j] = 0.f;
            }
        }
        if (more) {
            la.commit(sA[buf ^ 1]);
            lb.commit(sB[buf ^ 1]);
            __syncthreads();
            buf ^= 1;
        }
    }

    if constexpr (SPLITK) {
        __shared__ unsigned arrivedBefore;
        const unsigned tile = blockIdx.x + blockIdx.y * gridDim.x, tiles = gridDim.x * gridDim.y;
        constexpr int kPerTile = BM * BN;
        // element (i, j) of thread t at (i * TN + j) * kThreads + t: consecutive threads, consecutive addresses
        float* mine = g.partials + (size_t(blockIdx.z) * tiles + tile) * kPerTile;
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) mine[(i * TN + j) * kThreads + threadIdx.x] = acc[i][j];
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) arrivedBefore = atomicAdd(&g.counters[tile], 1u);
        __syncthreads();
        if (arrivedBefore + 1 < unsigned(g.splits)) return;
        __threadfence();  // the other slices' partial tiles are complete and visible
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
        for (int z = 0; z < g.splits; ++z) {  // slice order; the loads of one slice are independent of each other
            const float* part = g.partials + (size_t(z) * tiles + tile) * kPerTile + threadIdx.x;
            float v[TM][TN];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) v[i][j] = __ldcg(part + (i * TN + j) * kThreads);
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] += v[i][j];
        }
        if (threadIdx.x == 0) g.counters[tile] = 0;  // ready for the next call on this scratch memory
    }

    Epilogue<float> epi;
    epi.init(g.epi, entry);
#pragma unroll
    for (int j = 0; j < TN; ++j) {
        const int col = col0 + ty * 4 + (j / 4) * 64 + j % 4;
        if (col >= g.n) continue;
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int row = row0 + tx * 4 + (i / 4) * 64 + i % 4;
            if (row < g.m) epi.store(row, col, acc[i][j]);
        }
    }
}

template <int BM, int BN>
cudaError_t launchTile(const Problem& p, SgemmArgs& g, dim3 grid) {
    const bool am = !p.transA, bn = p.transB;
    if (am && bn) sgemmKernel<BM, BN, true, true><<<grid, kThreads, 0, p.stream>>>(g);
    else if (am) sgemmKernel<BM, BN, true, false><<<grid, kThreads, 0, p.stream>>>(g);
    else if (bn) sgemmKernel<BM, BN, false, true><<<grid, kThreads, 0, p.stream>>>(g);
    else sgemmKernel<BM, BN, false, false><<<grid, kThreads, 0, p.stream>>>(g);
    return cudaGetLastError();
}

constexpr int kMaxGridZ = 65535;

int smCountOnce() {
    static const int count = [] {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            n = 148;
        return n;
    }();
    return count;
}

}  // namespace

int sgemmSmCount() { return smCountOnce(); }

bool sgemmEligible(const Problem& p) {
    return p.accType == kF32 && p.typeA == kF32 && p.typeB == kF32 && !p.pointerArrays && p.k > 0 &&
           (reinterpret_cast<uintptr_t>(p.A) & 3) == 0 && (reinterpret_cast<uintptr_t>(p.B) & 3) == 0;
}

// Scratch memory of the split-k form: kSplitKCounters arrival counters (zero between calls), then the partial tiles.
size_t sgemmSplitKScratchBytes(int m, int n, int splits) {
    const size_t tiles = size_t((m + 63) / 64) * ((n + 63) / 64);
    return kSplitKCounters * sizeof(unsigned) + size_t(splits) * tiles * 64 * 64 * sizeof(float);
}

// How many slices of k a product should be cut into (1: do not split). Splitting pays when the 64 x 64 tiles alone leave
// most SMs idle and k is long enough to share out; the partial tiles must fit the scratch memory.
int sgemmSplitKPlan(const Problem& p, size_t scratchBytes) {
    if (p.batch != 1 || scratchBytes == 0) return 1;
    static const int forced = measureKnob("VKZB_SGEMM_SPLITS", 0);  // measurement builds only
    if (forced > 0) return sgemmSplitKScratchBytes(p.m, p.n, forced) <= scratchBytes && (long long)((p.m + 63) / 64) * ((p.n + 63) / 64) <= kSplitKCounters ? forced : 1;
    const long long tiles = (long long)((p.m + 63) / 64) * ((p.n + 63) / 64);
    if (tiles > kSplitKCounters || tiles * 2 > smCountOnce() || p.k < 256) return 1;  // measured: below k = 256 the hand-over costs more than it saves
    int splits = int(std::min<long long>(std::min<long long>(8, 2LL * smCountOnce() / tiles), p.k / 64));
    while (splits > 1 && sgemmSplitKScratchBytes(p.m, p.n, splits) > scratchBytes) --splits;
    return splits;
}

cudaError_t launchSgemmSplitK(const Problem& p, int splits, void* scratch) {
    SgemmArgs g{static_cast<const float*>(p.A), static_cast<const float*>(p.B), p.lda, p.ldb, 0, 0, p.m, p.n, p.k, 0, 0, p.epi};
    g.splits = splits;
    g.kPer = ((p.k + splits - 1) / splits + 15) / 16 * 16;  // whole shared-memory fills
    g.splits = (p.k + g.kPer - 1) / g.kPer;
    g.counters = static_cast<unsigned*>(scratch);
    g.partials = reinterpret_cast<float*>(g.counters + kSplitKCounters);
    const dim3 grid((p.m + 63) / 64, (p.n + 63) / 64, g.splits);
    const bool am = !p.transA, bn = p.transB;
    if (am && bn) sgemmKernel<64, 64, true, true, true><<<grid, kThreads, 0, p.stream>>>(g);
    else if (am) sgemmKernel<64, 64, true, false, true><<<grid, kThreads, 0, p.stream>>>(g);
    else if (bn) sgemmKernel<64, 64, false, true, true><<<grid, kThreads, 0, p.stream>>>(g);
    else sgemmKernel<64, 64, false, false, true><<<grid, kThreads, 0, p.stream>>>(g);
    countLaunch();
    return cudaGetLastError();
}

cudaError_t launchSgemm(const Problem& p) {
    if (p.scratch) {
        const int splits = sgemmSplitKPlan(p, p.scratchBytes);
        if (splits > 1) return launchSgemmSplitK(p, splits, p.scratch);
    }
    SgemmArgs g{static_cast<const float*>(p.A), static_cast<const float*>(p.B), p.lda, p.ldb, p.strideA, p.strideB,
                p.m, p.n, p.k, 0, 0, p.epi};
    // 128 x 128 tiles once they fill the machine; 64 x 64 below that so small products still spread over the SMs
    const long long bigTiles = (long long)((p.m + 127) / 128) * ((p.n + 127) / 128) * p.batch;
    const bool big = bigTiles >= smCountOnce();
    const int tile = big ? 128 : 64, tilesN = (p.n + tile - 1) / tile;
    for (int first = 0; first < p.batch; first += kMaxGridZ)
        for (int col = 0; col < tilesN; col += kMaxGridZ) {  // gridDim.y has the same limit as gridDim.z
            g.batchOffset = first, g.colTileBase = col;
            const unsigned gz = unsigned(std::min(p.batch - first, kMaxGridZ)), gy = unsigned(std::min(tilesN - col, kMaxGridZ));
            cudaError_t e;
            if (big) e = launchTile<128, 128>(p, g, dim3((p.m + 127) / 128, gy, gz));
            else e = launchTile<64, 64>(p, g, dim3((p.m + 63) / 64, gy, gz));
            countLaunch();
            if (e != cudaSuccess) return e;
        }
    return cudaSuccess;
}

}  // namespace vkzb
