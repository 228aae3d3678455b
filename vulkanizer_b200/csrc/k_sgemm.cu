// fp32 GEMM on the CUDA cores: register-blocked FFMA with float4-vectorised, coalesced global loads.
//
// Replaces k0zi/Vulkanizer's 128 x 128 tiled shader for fp32 operands (src/cublas/shaders/gemm_tiled.comp:178-240,
// selected at src/cublas/cublas.cpp:825-837): every transpose combination, 16-byte loads where pointer, leading
// dimension and tile offset allow, scalar loads at the ragged edges. A tile of op(A) and of op(B) is staged in
// shared memory k-major ([k][m] and [k][n]) so the inner product reads two float4 of each per k; the next k slice
// is fetched into registers while the current one is multiplied (two shared buffers, one barrier per slice).
// Accumulation is plain fp32 with k ascending, so results stay within 1e-5 of an fp64 reference.
#include "epilogue.cuh"

namespace vkzb {
namespace {

constexpr int kThreads = 256;

struct SgemmArgs {
    const float* A;
    const float* B;
    long long lda, ldb, strideA, strideB;
    int m, n, k;
    int batchOffset;
    EpilogueArgs epi;
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
template <int BM, int BN, bool A_MCONTIG, bool B_NCONTIG>
__global__ void __launch_bounds__(kThreads) sgemmKernel(const SgemmArgs g) {
    constexpr int TM = BM / 16, TN = BN / 16;        // 8 x 8 for 128 x 128, 4 x 4 for 64 x 64
    constexpr int GM = TM / 4, GN = TN / 4;          // float4 groups per thread
    constexpr int BK = BM >= 128 ? 8 : 16;           // k slice per shared-memory fill
    constexpr int kPitchA = BM + 4, kPitchB = BN + 4;
    __shared__ __align__(16) float sA[2][BK * kPitchA];
    __shared__ __align__(16) float sB[2][BK * kPitchB];

    const long long entry = (long long)blockIdx.z + g.batchOffset;
    const float* A = g.A + entry * g.strideA;
    const float* B = g.B + entry * g.strideB;
    const int row0 = blockIdx.x * BM, col0 = blockIdx.y * BN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;

    const bool vecA = (reinterpret_cast<uintptr_t>(A) & 15) == 0 && g.lda % 4 == 0;
    const bool vecB = (reinterpret_cast<uintptr_t>(B) & 15) == 0 && g.ldb % 4 == 0;

    TileLoader<BM, BK, A_MCONTIG> la;
    TileLoader<BN, BK, B_NCONTIG> lb;
    float acc[TM][TN] = {};

    la.fetch(A, g.lda, row0, g.m, 0, g.k, vecA);
    lb.fetch(B, g.ldb, col0, g.n, 0, g.k, vecB);
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
    for (int k0 = 0; k0 < g.k; k0 += BK) {
        const bool more = k0 + BK < g.k;
        if (more) {
            la.fetch(A, g.lda, row0, g.m, k0 + BK, g.k, vecA);
            lb.fetch(B, g.ldb, col0, g.n, k0 + BK, g.k, vecB);
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

int smCount() {
    static const int count = [] {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            n = 148;
        return n;
    }();
    return count;
}

}  // namespace

bool sgemmEligible(const Problem& p) {
    return p.accType == kF32 && p.typeA == kF32 && p.typeB == kF32 && !p.pointerArrays && p.k > 0 &&
           (reinterpret_cast<uintptr_t>(p.A) & 3) == 0 && (reinterpret_cast<uintptr_t>(p.B) & 3) == 0;
}

cudaError_t launchSgemm(const Problem& p) {
    SgemmArgs g{static_cast<const float*>(p.A), static_cast<const float*>(p.B), p.lda, p.ldb, p.strideA, p.strideB,
                p.m, p.n, p.k, 0, p.epi};
    // 128 x 128 tiles once they fill the machine; 64 x 64 below that so small products still spread over the SMs
    const long long bigTiles = (long long)((p.m + 127) / 128) * ((p.n + 127) / 128) * p.batch;
    const bool big = bigTiles >= smCount();
    for (int first = 0; first < p.batch; first += kMaxGridZ) {
        g.batchOffset = first;
        const unsigned gz = unsigned(std::min(p.batch - first, kMaxGridZ));
        cudaError_t e;
        if (big) e = launchTile<128, 128>(p, g, dim3((p.m + 127) / 128, (p.n + 127) / 128, gz));
        else e = launchTile<64, 64>(p, g, dim3((p.m + 63) / 64, (p.n + 63) / 64, gz));
        countLaunch();
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace vkzb
