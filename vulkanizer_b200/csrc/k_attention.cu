// vkzbAttentionForward: O = softmax(scale Q K^T + mask) V in one kernel, for f16 / bf16 and head dimensions 64 and 128.
//
// What it replaces: the batched product Q K^T (the benchmark's batched-attention shape) writes batch x numQ x numK scores to
// memory (1 GiB of fp32 for 256 heads of 1024 x 1024), a softmax pass reads and writes them again and a second batched
// product reads them a third time. Here a CTA owns 256 queries of one head, as two tiles of 128, and walks the keys in tiles
// of 128: scores and probabilities live in tensor memory only, and what reaches HBM is Q, K, V once (K and V once per CTA,
// from L2) and O.
//
// Roles in a CTA of 320 threads (the scheme of the GEMM kernel in k_umma.cu, with the two-tile alternation of FlashAttention-4):
//   warp 0      one lane issues the TMA loads: the two Q tiles once, then K and V tiles through two-stage rings;
//   warp 1      one elected lane issues tcgen05.mma. Tensor memory holds S and O of both query tiles (4 x 128 columns). Per
//               key tile and query tile t: S_t = Q_t K_j^T; and, when the probabilities are there, O_t += P_t V_j with P_t
//               read from tensor memory (it overlays S_t). While the softmax warps of one query tile work on their scores
//               the tensor cores run the other tile's products;
//   warps 2-5 and 6-9   query tile 0 and 1, one thread per query row: read the row of S, keep the running maximum and sum
//               (the online softmax of Milakov and Gimelshein, as used by FlashAttention), write P as 16-bit pairs over the
//               columns of S already read, rescale the row of O when the maximum moved far, and at the end divide by the
//               sum and put the row into the query tile's shared memory, from where a bulk tensor store takes the tile.
// What was measured and dropped (256 heads of 1024 x 1024 x 128, f16): steps of 64 keys with S, P and O in columns of their
// own, so that no product waits for the exponentials (S products of 64 columns read Q from shared memory again for half the
// work: 186 us against 155); two exponentials per special-function instruction in 16 bits (three times slower); a cubic
// on the FMA pipe for a quarter of the exponentials (slower), fp32 arithmetic on pairs in that loop (no change), the two tiles
// taking turns at the special-function unit (slightly slower); CTAs that
// walk several work items, statically dealt or drawn from a counter (149 - 166 us, and worse under a causal mask); P through
// shared memory instead of tensor memory, so that a tile's next scores are computed before its P V and its softmax warps
// start half a product earlier (188 us: both products then read both operands from shared memory, which the softmax warps'
// stores and the loads also use); the maximum taken inside the exponential pass against the row's previous reference point,
// with a second pass only when it moved by more than 2^8 (163 us: that loop is the bottleneck, and the extra maxima and the
// held-back probabilities cost it more than the separate pass did).
// Every wait is bounded: a wait that runs out records a code in g_attentionStatus, raises the CTA's abort flag and all
// roles leave through the common exit, which frees the tensor memory.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <mutex>
#include <type_traits>

#include "../../include/vkzb_attention.h"
#include "gemm_problem.h"

namespace vkzb {
namespace {

constexpr int kTileQ = 128;                 // queries per CTA = TMEM lanes
constexpr int kTileK = 128;                 // keys per step
constexpr int kQueriesPerCta = 256;         // two query tiles share the K and V tiles a CTA loads
constexpr int kAttnThreads = 320;           // loader, issuer, four softmax warps per query tile
constexpr int kAtomBytes = 128 * 128;       // 128 rows of one 128-byte swizzle span
constexpr int kVBoxBytes = 64 * 128;        // 64 keys x 64 values of V
constexpr unsigned long long kAttnWaitLimitNs = 4000000000ull;
constexpr unsigned kTmemColumns = 512;      // S and O of two query tiles, 128 columns each

enum : unsigned { kAttnOk = 0, kAttnProducerWait = 33, kAttnMmaWait = 34, kAttnSoftmaxWait = 35 };
__device__ unsigned g_attentionStatus;

struct AttentionArgs {
    int numQ, numK, heads, kvGroup;
    int mask;            // 0 none, 1 causal from the top left, 2 from the bottom right
    float scaleLog2;     // scale * log2(e): the exponentials are taken in base 2
    float* logSumExp;    // [batch][head][numQ], or null
    unsigned idescS, idescO;
};

// ---- PTX wrappers (the same instructions as in k_umma.cu; this file is a translation unit of its own) -----------------

__device__ __forceinline__ unsigned smemAddr(const void* p) { return unsigned(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbarInit(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarArriveExpectTx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarArrive(unsigned bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool mbarTryWait(unsigned bar, unsigned parity) {
    unsigned done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return done != 0;
}
__device__ __forceinline__ unsigned long long globalTimerNs() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// False when the CTA is aborting or the wait ran out of time (the code is then recorded and the abort flag raised).
__device__ __noinline__ bool mbarWaitSlow(unsigned bar, unsigned parity, volatile int* abortFlag, unsigned code) {
    const unsigned long long start = globalTimerNs();
    for (unsigned spins = 0;; ++spins) {
        if (mbarTryWait(bar, parity)) return true;
        if ((spins & 63u) == 63u) {
            if (*abortFlag) return false;
            if (globalTimerNs() - start > kAttnWaitLimitNs) {
                atomicCAS(&g_attentionStatus, kAttnOk, code);
                *abortFlag = 1;
                __threadfence_block();
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbarWait(unsigned bar, unsigned parity, volatile int* abortFlag, unsigned code) {
    if (mbarTryWait(bar, parity)) return true;
    return mbarWaitSlow(bar, parity, abortFlag, code);
}
__device__ __forceinline__ void tmaLoad4d(unsigned dst, const CUtensorMap* map, unsigned bar, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<unsigned long long>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
// Shared memory -> global, asynchronous; rows outside the tensor are clipped by the hardware.
__device__ __forceinline__ void tmaStore4d(const CUtensorMap* map, unsigned src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(reinterpret_cast<unsigned long long>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ bool electOne() {
    unsigned elected;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(elected));
    return elected != 0;
}
__device__ __forceinline__ void tcgen05FenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05FenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05Commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mmaF16(unsigned tmemD, unsigned long long descA, unsigned long long descB, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// The same with A (the probabilities) read from tensor memory: row i in lane i, two 16-bit values of k per 32-bit column.
__device__ __forceinline__ void mmaF16FromTmem(unsigned tmemD, unsigned tmemA, unsigned long long descB, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmemD), "r"(tmemA), "l"(descB), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// Generic-proxy writes to shared memory before, asynchronous-proxy reads (the tensor cores') after.
__device__ __forceinline__ void fenceAsyncShared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// 32 lanes x 32 columns of 32-bit cells: thread i of the warp receives row i.
__device__ __forceinline__ void tmemLoad32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmemStore32(unsigned taddr, const unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
        "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmemLoad32Issue(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmemWaitLoads() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmemStore16Issue(unsigned taddr, const unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmemWaitStores() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// sm_100's three-input maximum
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float exp2Approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
template <bool BF16>
__device__ __forceinline__ unsigned packPair(float lo, float hi) {
    if constexpr (BF16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const unsigned*>(&v);
    } else {
        const __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const unsigned*>(&v);
    }
}

// Shared-memory plan for head dimension D (elements of 2 bytes). Q and K tiles: D / 64 atoms of 128 rows x 128 bytes
// (64 values of the head dimension per row: the K-major operand layout under the 128-byte swizzle). V tiles: the
// head dimension is the contiguous one and is the N side of the second product, so V is staged as boxes of 64 keys x 64
// values, ordered [half of the keys][chunk of the head dimension]. Two query tiles, two stages of K, two of V.
template <int D>
struct AttnPlan {
    static constexpr int kAtoms = D / 64;
    static constexpr int kTileBytes = kAtoms * kAtomBytes;       // a Q or K tile
    static constexpr int kVBytes = 2 * kAtoms * kVBoxBytes;      // a V tile: the same size
    static constexpr int kOffK = 2 * kTileBytes;
    static constexpr int kOffV = kOffK + 2 * kTileBytes;
    static constexpr int kOffBars = kOffV + 2 * kVBytes;
    static constexpr int kUsedBytes = kOffBars + 256 + 1024;     // barriers and flags; slack to align the base to 1024 bytes
    // a CTA takes all 512 columns of tensor memory, so a second CTA on the SM could only wait for it: ask for more than
    // half of the SM's shared memory even where the tiles need less
    static constexpr int kSmemBytes = kUsedBytes > 120 * 1024 ? kUsedBytes : 120 * 1024;
};

// Barrier numbers (8 bytes each from the start of the barrier block); [2] = one per query tile or per stage.
enum : unsigned { kBarQ = 0, kBarKFull = 2, kBarKEmpty = 4, kBarVFull = 6, kBarVEmpty = 8, kBarS = 10, kBarP = 12, kBarO = 14, kBarCount = 16 };

template <int D, bool BF16>
__global__ void __launch_bounds__(kAttnThreads, 1)
attentionKernel(const AttentionArgs g, const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapO) {
    using Plan = AttnPlan<D>;
    constexpr int kAtoms = Plan::kAtoms;
    extern __shared__ unsigned char smemRaw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + Plan::kOffBars);
    unsigned* tmemSlot = reinterpret_cast<unsigned*>(bars + kBarCount);
    volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const unsigned base = smemAddr(smem);
    const unsigned bar0 = smemAddr(bars);
    const auto bar = [&](unsigned which, int index) { return bar0 + 8 * (which + unsigned(index)); };
    // under a causal mask the later queries have more keys to visit: their CTAs start first, so the short ones fill the tail
    const int q0 = int(g.mask ? gridDim.x - 1 - blockIdx.x : blockIdx.x) * kQueriesPerCta, head = blockIdx.y, batch = blockIdx.z;
    const int kvHead = head / g.kvGroup;
    // keys a query may see: index <= query + diag
    const int diag = g.mask == 2 ? g.numK - g.numQ : 0;
    // key tiles that hold a key some query of query tile t may see
    const auto keyTilesOf = [&](int t) {
        const int first = q0 + t * kTileQ;
        if (first >= g.numQ) return 0;
        const int lastQuery = min(first + kTileQ, g.numQ) - 1;
        const int reach = g.mask ? max(0, min(g.numK, lastQuery + diag + 1)) : g.numK;
        return (reach + kTileK - 1) / kTileK;
    };
    const int tiles[2] = {keyTilesOf(0), keyTilesOf(1)};
    const int steps = max(tiles[0], tiles[1]);

    const auto loadQ = [&](int t) {
        mbarArriveExpectTx(bar(kBarQ, t), Plan::kTileBytes);
        for (int a = 0; a < kAtoms; ++a) tmaLoad4d(base + t * Plan::kTileBytes + a * kAtomBytes, &mapQ, bar(kBarQ, t), 64 * a, q0 + t * kTileQ, head, batch);
    };
    const auto loadK = [&](int j) {
        const int stage = j & 1;
        mbarArriveExpectTx(bar(kBarKFull, stage), Plan::kTileBytes);
        for (int a = 0; a < kAtoms; ++a)
            tmaLoad4d(base + Plan::kOffK + stage * Plan::kTileBytes + a * kAtomBytes, &mapK, bar(kBarKFull, stage), 64 * a, j * kTileK, kvHead, batch);
    };
    const auto loadV = [&](int j) {
        const int stage = j & 1;
        mbarArriveExpectTx(bar(kBarVFull, stage), Plan::kVBytes);
        for (int half = 0; half < 2; ++half)
            for (int c = 0; c < kAtoms; ++c)
                tmaLoad4d(base + Plan::kOffV + stage * Plan::kVBytes + (half * kAtoms + c) * kVBoxBytes, &mapV, bar(kBarVFull, stage), 64 * c,
                          j * kTileK + 64 * half, kvHead, batch);
    };
    if (threadIdx.x == 0) {
        for (unsigned b = 0; b < kBarCount; ++b) mbarInit(bar0 + 8 * b, b == kBarP || b == kBarP + 1 ? 4 : 1);  // P: one arrival per softmax warp
        *abortFlag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fenceAsyncShared();
        // This thread is also the loader: the first tiles are on their way while the tensor memory is still being
        // allocated, in the order the first products need them (both stages are free, so nothing to wait for).
        if (steps > 0) {
            if (tiles[0]) loadQ(0);
            loadK(0);
            if (tiles[1]) loadQ(1);
            loadV(0);
            if (steps > 1) loadK(1), loadV(1);
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(tmemSlot)), "r"(kTmemColumns) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05FenceBefore();
    __syncthreads();
    tcgen05FenceAfter();
    const unsigned tmemBase = *tmemSlot;
    // columns: S of query tile 0 | S of tile 1 | O of tile 0 | O of tile 1; P of a tile overlays the first 64 columns of its S

    if (warp == 0) {
        // ---- TMA producer ----
        if (lane == 0) {
            for (int j = 2; j < steps; ++j) {  // tiles 0 and 1 were requested during set-up
                const int stage = j & 1;
                const unsigned freed = ((j >> 1) & 1) ^ 1;
                if (!mbarWait(bar(kBarKEmpty, stage), freed, abortFlag, kAttnProducerWait)) break;
                loadK(j);
                if (!mbarWait(bar(kBarVEmpty, stage), freed, abortFlag, kAttnProducerWait)) break;
                loadV(j);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---- MMA issuer ----
        // The tensor cores run what this lane issues in order, so S_t of the next key tile may be issued right behind the
        // P V of this one although both use the same columns. Per key tile and query tile: wait for the probabilities, issue
        // O_t += P_t V, issue S_t of the next key tile. While the softmax warps of one query tile work, the tensor cores run
        // the other tile's products.
        // shared-memory descriptors: stride offset 1024 bytes (8 rows of 128 bytes), version 1, 128-byte swizzle; the leading
        // offset is unused for K-major operands (1) and the distance between 64-value chunks for V
        const unsigned long long hi = static_cast<unsigned long long>((1024u >> 4) | 1u << 14 | 2u << 29) << 32;
        const auto desc = [&](unsigned addr, unsigned lbo) { return hi | (((addr & 0x3FFFFu) >> 4) | lbo << 16); };
        // the whole warp takes every decision together: a wait that gave up in one lane ends the loop for all
        const auto waitAll = [&](unsigned b, unsigned parity) { return __all_sync(0xFFFFFFFFu, mbarWait(b, parity, abortFlag, kAttnMmaWait)) != 0; };
        const auto issueS = [&](int t, int j) {  // S_t = Q_t K_j^T, 16 values of the head dimension per instruction
            const int stage = j & 1;
#pragma unroll
            for (int a = 0; a < kAtoms; ++a) {
                const unsigned long long dq = desc(base + t * Plan::kTileBytes + a * kAtomBytes, 1);
                const unsigned long long dk = desc(base + Plan::kOffK + stage * Plan::kTileBytes + a * kAtomBytes, 1);
#pragma unroll
                for (int q = 0; q < 4; ++q) mmaF16(tmemBase + 128 * t, dq + 2 * q, dk + 2 * q, g.idescS, (a | q) ? 1u : 0u);
            }
            tcgen05Commit(bar(kBarS, t));
        };
        const auto issuePV = [&](int t, int j) {  // O_t += P_t V_j, 16 keys per instruction: 8 columns of P (two values each)
            const int stage = j & 1;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const unsigned long long dv = desc(base + Plan::kOffV + stage * Plan::kVBytes + half * kAtoms * kVBoxBytes, kVBoxBytes >> 4);
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    mmaF16FromTmem(tmemBase + 256 + 128 * t, tmemBase + 128 * t + 8 * (4 * half + q), dv + q * (2048 >> 4), g.idescO, (j | half | q) ? 1u : 0u);
            }
            tcgen05Commit(bar(kBarO, t));
        };
        bool ok = steps == 0 || waitAll(bar(kBarKFull, 0), 0);
        for (int t = 0; ok && t < 2; ++t) {
            if (!tiles[t]) continue;
            if (!(ok = waitAll(bar(kBarQ, t), 0))) break;
            tcgen05FenceAfter();
            if (electOne()) issueS(t, 0);
            __syncwarp();
        }
        if (ok && steps > 0 && electOne()) tcgen05Commit(bar(kBarKEmpty, 0));  // K tile 0 has no reader left once these products are done
        __syncwarp();
        for (int j = 0; ok && j < steps; ++j) {
            const int stage = j & 1, next = stage ^ 1;
            if (!(ok = waitAll(bar(kBarVFull, stage), (j >> 1) & 1))) break;
            if (j + 1 < steps && !(ok = waitAll(bar(kBarKFull, next), ((j + 1) >> 1) & 1))) break;
            for (int t = 0; ok && t < 2; ++t) {
                if (j >= tiles[t]) continue;
                if (!(ok = waitAll(bar(kBarP, t), j & 1))) break;
                tcgen05FenceAfter();
                if (electOne()) {
                    issuePV(t, j);
                    if (j + 1 < tiles[t]) issueS(t, j + 1);
                }
                __syncwarp();
            }
            if (ok && electOne()) {
                tcgen05Commit(bar(kBarVEmpty, stage));                      // every P V of this key tile has been issued
                if (j + 1 < steps) tcgen05Commit(bar(kBarKEmpty, next));    // and every S of the next one
            }
            __syncwarp();
        }
    } else {
        // ---- softmax and output: four warps per query tile, one thread per query ----
        const int t = (warp - 2) / 4;
        const int quarter = warp % 4;  // a warp may only touch TMEM lanes 32 * (warp % 4) .. + 31
        const int rowInTile = quarter * 32 + lane, query = q0 + t * kTileQ + rowInTile;
        const unsigned laneBits = unsigned(quarter * 32) << 16;
        const unsigned tmemS = tmemBase + 128 * t + laneBits, tmemO = tmemBase + 256 + 128 * t + laneBits;
        const int visible = g.mask ? max(0, min(g.numK, query + diag + 1)) : g.numK;  // keys [0, visible) count for this row
        const int myTiles = tiles[t];
        const float c = g.scaleLog2;
        float runMax = -INFINITY, runSum = 0.f;
        // tcgen05.ld and .st are warp-wide: the warp takes every decision together
        const auto waitAll = [&](unsigned b, unsigned parity) { return __all_sync(0xFFFFFFFFu, mbarWait(b, parity, abortFlag, kAttnSoftmaxWait)) != 0; };
        bool ok = true;
        for (int j = 0; j < myTiles; ++j) {
            // S_t of this key tile is complete, and with it everything issued before it: the previous P V has read P and updated O
            if (!(ok = waitAll(bar(kBarS, t), j & 1))) break;
            tcgen05FenceAfter();
            const int limit = visible - j * kTileK;  // columns [0, limit) of this tile count
            // the same code path for the whole warp (tcgen05.ld and .st must not sit in a branch that lanes take differently)
            const bool allCount = __all_sync(0xFFFFFFFFu, limit >= kTileK) != 0;
            // the whole row of S in registers: four loads in flight, one wait
            unsigned v[kTileK];
#pragma unroll
            for (int chunk = 0; chunk < 4; ++chunk) tmemLoad32Issue(tmemS + 32 * chunk, *reinterpret_cast<unsigned(*)[32]>(v + 32 * chunk));
            tmemWaitLoads();
            float tileMax = -INFINITY;
            if (allCount && c >= 0.f) {
                // every column counts: the maximum of the raw scores (three at a time), scaled once
                float m[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) m[i] = fmaxf(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
#pragma unroll
                for (int i = 16; i < kTileK; i += 16)
#pragma unroll
                    for (int a = 0; a < 8; ++a) m[a] = max3(m[a], __uint_as_float(v[i + 2 * a]), __uint_as_float(v[i + 2 * a + 1]));
                tileMax = max3(max3(m[0], m[1], m[2]), max3(m[3], m[4], m[5]), fmaxf(m[6], m[7])) * c;
            } else {
#pragma unroll
                for (int i = 0; i < kTileK; ++i)
                    if (i < limit) tileMax = fmaxf(tileMax, __uint_as_float(v[i]) * c);
            }
            // The reference point of the exponentials moves only when the maximum has grown by more than 2^8: until then the
            // probabilities are at most 256 (exact enough in 16 bits, far from overflow in the sums) and the row of O needs
            // no rescaling. The final division by the sum, taken against the same reference point, makes the result the same.
            const float newMax = runMax == -INFINITY || tileMax > runMax + 8.f ? tileMax : runMax;
            const float shift = newMax == -INFINITY ? 0.f : newMax;  // a row that has seen no key yet
            const float correction = newMax == runMax ? 1.f : exp2Approx(runMax - shift);  // 0 for the first keys of a row
            runMax = newMax;
            // exp2(c s - shift) on the special-function unit (16 results per clock and SM)
            const float negShift = -shift;
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
            // The row is read a second time, 32 columns at a time with the next 32 already on their way: holding all 128 scores
            // through this loop leaves the compiler too few registers to keep enough exponentials in flight.
            unsigned ping[32], pong[32];
            const auto exponentials = [&](const unsigned (&s32)[32], int chunk) {
                unsigned packed[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int col = chunk * 32 + 2 * i;
                    const float x0 = fmaf(__uint_as_float(s32[2 * i]), c, negShift), x1 = fmaf(__uint_as_float(s32[2 * i + 1]), c, negShift);
                    float p0 = exp2Approx(x0), p1 = exp2Approx(x1);
                    if (!allCount) p0 = col < limit ? p0 : 0.f, p1 = col + 1 < limit ? p1 : 0.f;
                    sum[i & 3] += p0 + p1;
                    packed[i] = packPair<BF16>(p0, p1);
                }
                // P overlays S: columns 16 chunk .. + 15 of the row, behind everything still to be read
                tmemStore16Issue(tmemS + 16 * chunk, packed);
            };
            tmemLoad32Issue(tmemS, ping);
            tmemWaitLoads();
            tmemLoad32Issue(tmemS + 32, pong);
            exponentials(ping, 0);
            tmemWaitLoads();
            tmemLoad32Issue(tmemS + 64, ping);
            exponentials(pong, 1);
            tmemWaitLoads();
            tmemLoad32Issue(tmemS + 96, pong);
            exponentials(ping, 2);
            tmemWaitLoads();
            exponentials(pong, 3);
            const float tileSum = (sum[0] + sum[1]) + (sum[2] + sum[3]);
            tmemWaitStores();
            runSum = runSum * correction + tileSum;
            if (j > 0 && __any_sync(0xFFFFFFFFu, correction != 1.f)) {
#pragma unroll
                for (int chunk = 0; chunk < D / 32; ++chunk) {
                    unsigned o[32];
                    tmemLoad32(tmemO + 32 * chunk, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * correction);
                    tmemStore32(tmemO + 32 * chunk, o);
                }
            }
            tcgen05FenceBefore();
            __syncwarp();
            if (lane == 0) mbarArrive(bar(kBarP, t));
        }
        if (ok && myTiles > 0) ok = waitAll(bar(kBarO, t), (myTiles - 1) & 1);
        tcgen05FenceAfter();
        // The rows of O leave through the query tile's shared memory (free once the last S has been computed) and two bulk
        // tensor stores: a thread holds a whole row, so direct stores would touch 32 rows with every instruction.
        if (ok) {
            const float inverse = runSum > 0.f ? 1.f / runSum : 0.f;
            unsigned char* rowBase = smem + t * Plan::kTileBytes + rowInTile * 128;
            // the whole row at once: all the loads in flight, one wait (nothing else is alive in registers by now)
            unsigned v[D];
            if (myTiles > 0) {
#pragma unroll
                for (int chunk = 0; chunk < D / 32; ++chunk) tmemLoad32Issue(tmemO + 32 * chunk, *reinterpret_cast<unsigned(*)[32]>(v + 32 * chunk));
                tmemWaitLoads();
            } else {
#pragma unroll
                for (int i = 0; i < D; ++i) v[i] = 0u;
            }
#pragma unroll
            for (int index = 0; index < D / 8; ++index) {
                unsigned w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    w[i] = packPair<BF16>(__uint_as_float(v[8 * index + 2 * i]) * inverse, __uint_as_float(v[8 * index + 2 * i + 1]) * inverse);
                // 16-byte piece `index` of the row: atom (index / 8), position (index % 8) ^ (row % 8), as TMA expects it
                *reinterpret_cast<uint4*>(rowBase + (index / 8) * kAtomBytes + (((index % 8) ^ (rowInTile & 7)) * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            if (g.logSumExp && query < g.numQ)  // natural logarithm of the sum of exp(score); 0 for a row without visible keys
                g.logSumExp[(size_t(batch) * g.heads + head) * g.numQ + query] = runSum > 0.f ? (runMax + log2f(runSum)) * 0.6931471805599453f : 0.f;
        }
        // every warp of the tile comes here, whatever happened before: the barrier must not wait for a warp that gave up
        fenceAsyncShared();
        if (t == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
        else asm volatile("bar.sync 2, 128;" ::: "memory");
        if (rowInTile == 0 && *abortFlag == 0 && q0 + t * kTileQ < g.numQ) {
            for (int a = 0; a < kAtoms; ++a) tmaStore4d(&mapO, base + t * Plan::kTileBytes + a * kAtomBytes, 64 * a, q0 + t * kTileQ, head, batch);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the shared memory is read before the CTA may end
        }
    }

    // ---- common exit ----
    if (*abortFlag) __nanosleep(20000);  // let copies still in flight land before the shared memory is released
    tcgen05FenceBefore();
    __syncthreads();
    if (warp == 1) {
        tcgen05FenceAfter();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(kTmemColumns) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encodeTiled() {
    static const EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// (value of the head dimension, position in the sequence, head, batch entry); strides in elements.
bool encodeSequence(CUtensorMap* map, const void* base, bool bf16, int headDim, int length, int heads, int batches, long long row, long long head,
                    long long batch, unsigned boxRows) {
    const cuuint64_t dims[4] = {cuuint64_t(headDim), cuuint64_t(length), cuuint64_t(heads), cuuint64_t(batches)};
    // a dimension of extent 1 still needs a legal stride (a multiple of 16 bytes): its value is never used
    const cuuint64_t strides[3] = {cuuint64_t(row) * 2, heads > 1 ? cuuint64_t(head) * 2 : cuuint64_t(row) * 2, batches > 1 ? cuuint64_t(batch) * 2 : cuuint64_t(row) * 2};
    const cuuint32_t box[4] = {64, boxRows, 1, 1};
    const cuuint32_t elemStrides[4] = {1, 1, 1, 1};
    return encodeTiled()(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box,
                         elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D, bool BF16>
cudaError_t launchAttention(const AttentionArgs& g, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo, dim3 grid,
                            cudaStream_t stream) {
    static std::mutex mutex;
    static bool attributeSet[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    device = device < 0 || device >= 64 ? 0 : device;
    {
        std::lock_guard<std::mutex> lock(mutex);
        if (!attributeSet[device]) {
            const cudaError_t e = cudaFuncSetAttribute(attentionKernel<D, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnPlan<D>::kSmemBytes);
            if (e != cudaSuccess) return e;
            attributeSet[device] = true;
        }
    }
    attentionKernel<D, BF16><<<grid, kAttnThreads, AttnPlan<D>::kSmemBytes, stream>>>(g, mq, mk, mv, mo);
    countLaunch();
    return cudaGetLastError();
}

}  // namespace
}  // namespace vkzb

extern "C" __attribute__((visibility("default"))) int vkzbAttentionForward(cudaStream_t stream, const vkzbAttentionProblem* a) {
    using namespace vkzb;
    enum { kSuccess = 0, kNotInitialized = 1, kInvalidValue = 7, kExecutionFailed = 13, kNotSupported = 15 };  // cublasStatus_t values
    if (!a || a->batches < 0 || a->heads < 0 || a->kvHeads <= 0 || a->numQ < 0 || a->numK < 0 || unsigned(a->mask) > 2u) return kInvalidValue;
    if (a->heads % a->kvHeads) return kInvalidValue;
    if (a->dataType != 2 /* CUDA_R_16F */ && a->dataType != 14 /* CUDA_R_16BF */) return kNotSupported;
    if (a->headDim != 64 && a->headDim != 128) return kNotSupported;
    if (a->batches == 0 || a->heads == 0 || a->numQ == 0) return kSuccess;
    if (!a->q || !a->k || !a->v || !a->o) return kInvalidValue;
    if (a->heads > 65535 || a->batches > 65535) return kNotSupported;
    // TMA and the 16-byte stores of O: every base and every stride a multiple of 16 bytes
    const long long strides[] = {a->qRow, a->qHead, a->qBatch, a->kRow, a->kHead, a->kBatch, a->vRow, a->vHead, a->vBatch, a->oRow, a->oHead, a->oBatch};
    for (long long s : strides)
        if (s < 0 || s % 8) return kNotSupported;
    if (a->qRow < a->headDim || a->kRow < a->headDim || a->vRow < a->headDim || a->oRow < a->headDim) return kInvalidValue;
    for (const void* p : {a->q, a->k, a->v, static_cast<const void*>(a->o)})
        if (reinterpret_cast<uintptr_t>(p) % 16) return kNotSupported;
    if (!encodeTiled()) return kNotInitialized;
    const bool bf16 = a->dataType == 14;
    const int numK = a->numK;
    CUtensorMap mq, mk, mv, mo;
    // with no keys the kernel loads nothing; the maps still have to describe some memory, so they get extent 1
    if (!encodeSequence(&mq, a->q, bf16, a->headDim, a->numQ, a->heads, a->batches, a->qRow, a->qHead, a->qBatch, kTileQ) ||
        !encodeSequence(&mk, a->k, bf16, a->headDim, numK > 0 ? numK : 1, a->kvHeads, a->batches, a->kRow, a->kHead, a->kBatch, kTileK) ||
        !encodeSequence(&mv, a->v, bf16, a->headDim, numK > 0 ? numK : 1, a->kvHeads, a->batches, a->vRow, a->vHead, a->vBatch, 64) ||
        !encodeSequence(&mo, a->o, bf16, a->headDim, a->numQ, a->heads, a->batches, a->oRow, a->oHead, a->oBatch, kTileQ))
        return kNotSupported;
    AttentionArgs g{};
    g.numQ = a->numQ, g.numK = numK, g.heads = a->heads, g.kvGroup = a->heads / a->kvHeads;
    g.mask = a->mask;
    g.scaleLog2 = a->scale * 1.4426950408889634f;
    g.logSumExp = a->logSumExp;
    const unsigned format = bf16 ? 1u : 0u;
    // accumulate in f32; A and B in `format`; M = 128; S: N = 128 keys, both operands K-major; O: N = head dimension, B (V) N-major
    g.idescS = 1u << 4 | format << 7 | format << 10 | unsigned(kTileK >> 3) << 17 | unsigned(kTileQ >> 4) << 24;
    g.idescO = 1u << 4 | format << 7 | format << 10 | 1u << 16 | unsigned(a->headDim >> 3) << 17 | unsigned(kTileQ >> 4) << 24;
    const dim3 grid(unsigned((a->numQ + kQueriesPerCta - 1) / kQueriesPerCta), unsigned(a->heads), unsigned(a->batches));
    cudaError_t e;
    if (a->headDim == 128) e = bf16 ? launchAttention<128, true>(g, mq, mk, mv, mo, grid, stream) : launchAttention<128, false>(g, mq, mk, mv, mo, grid, stream);
    else e = bf16 ? launchAttention<64, true>(g, mq, mk, mv, mo, grid, stream) : launchAttention<64, false>(g, mq, mk, mv, mo, grid, stream);
    return e == cudaSuccess ? kSuccess : kExecutionFailed;
}

extern "C" __attribute__((visibility("default"))) int vkzbAttentionStatus(void) {
    unsigned status = 0;
    if (cudaMemcpyFromSymbol(&status, vkzb::g_attentionStatus, sizeof status) != cudaSuccess) return -1;
    return int(status);
}
