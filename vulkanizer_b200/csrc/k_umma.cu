// Tensor-core GEMM for Blackwell (sm_100a): TMA -> shared memory -> tcgen05.mma -> TMEM -> fused epilogue.
//
// This is the B200 counterpart of k0zi/Vulkanizer's cooperative-matrix shader (src/cublas/shaders/gemm_coopmat.comp:349-464,
// chosen at src/cublas/cublas.cpp:791-901) and of its f16 A^T B shader (gemm_f16_tn.comp:183-223): f16 or bf16
// operands with fp32 accumulation in every transpose combination, C in f32 / f16 / bf16, alpha and beta fused into
// the store. Beyond the reference it also covers int8 operands with exact int32 accumulation (kind::i8) and fp32
// operands on TF32 tensor cores (kind::tf32, only when the caller asked for TF32 math).
//
// One persistent CTA per SM walks output tiles of 128 x BN (BN = 256, 128 or 64) in a grouped order that keeps a
// band of A panels and the B panels they meet resident in L2 (the same idea as gemm_coopmat.comp:353-360). Warps
// are specialised:
//   warp 0    one lane issues the TMA loads of A and B k-slices into a ring of shared-memory stages
//   warp 1    one lane issues tcgen05.mma for each filled stage; accumulators live in TMEM, two of them,
//             so the next tile's products start while the previous tile is still being written out
//   warps 2-9 two groups of four; each warp reads its 32 TMEM lanes (= 32 rows of the tile) with tcgen05.ld, the
//             groups taking alternate column steps, and D = act(alpha * acc + beta * C + bias) leaves either through
//             a shared-memory buffer and a TMA bulk store (16-byte aligned D) or as direct column-major stores: for
//             a fixed column the 32 lanes of a warp touch 32 consecutive rows, i.e. one full 128-byte line
// A k-slice is 128 bytes per row (64 halves, 32 floats or 128 int8) so that TMA's 128-byte swizzle and the
// matrix descriptors' SWIZZLE_128B layout agree. Operands that are contiguous along k ("K-major": op(A) = A^T,
// op(B) = B) arrive as one box of rows x 128 bytes; operands contiguous along m or n ("MN-major") arrive as
// boxes of 128 bytes (of m or n) x slice-length rows, and the descriptor's leading-dimension byte offset steps
// between those boxes. Rows, columns and the k tail that fall outside the matrices are zero-filled by TMA.
//
// Every wait on an mbarrier is bounded in time: when one gives up it records a code in a device status
// word, raises a CTA-wide abort flag, and all roles fall through to the common exit, which frees TMEM.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "epilogue.cuh"
#include "measure.h"

namespace vkzb {
namespace {

constexpr int kBM = 128;                    // tile rows = TMEM lanes
constexpr int kSliceBytes = 128;            // bytes of k per row and stage (one swizzle span)
constexpr int kStageABytes = kBM * kSliceBytes;
constexpr int kMmasPerStage = 4;            // 128 bytes / 32 bytes of k per tcgen05.mma
constexpr int kEpilogueGroups = 2;             // each group of 4 warps covers the 128 TMEM lanes and takes every other column step
constexpr int kEpilogueWarps = 4 * kEpilogueGroups;
constexpr int kThreads = 32 * (2 + kEpilogueWarps);
constexpr int kSmemTotal = 227 * 1024;      // dynamic shared memory a CTA may have on sm_100
constexpr int kStoreCols = 16;                // columns per chunk of the split hand-over
constexpr int kStagingBufferBytes = kBM * kStoreCols * 4;             // the unit of epilogue staging memory: 128 rows x 16 columns of 4 bytes
constexpr unsigned long long kWaitLimitNs = 4000000000ull;  // a wait longer than this is a lost signal

enum UmmaKind : int { kKindF16 = 0, kKindTf32 = 1, kKindI8 = 2 };

// Codes left in the device status word by the wait that gave up.
enum : unsigned { kStatusOk = 0, kStatusProducerWait = 1, kStatusMmaFullWait = 2, kStatusMmaTmemWait = 3, kStatusEpilogueWait = 4 };

__device__ unsigned g_ummaStatus;

// Tensor maps of the buffers that receive a copy of every D tile (same shape and strides as D's map).
struct MirrorMaps {
    CUtensorMap map[kMaxMirrors];
};

struct UmmaArgs {
    int m, n, k, batch;
    int tilesM, tilesN, groupM;
    long long totalTiles;
    int numKSlices;   // ceil(k / sliceElems)
    int sliceElems;   // elements of k per stage: 128 bytes / element size
    int kind;         // UmmaKind
    unsigned idesc;   // tcgen05 instruction descriptor
    unsigned descHi;  // upper half of both shared-memory descriptors: stride offset, version, swizzle mode
    unsigned lboA, lboB;            // leading-dimension byte offset >> 4
    unsigned kStepA, kStepB;        // descriptor start-address advance per MMA, in 16-byte units
    int mnMajorA, mnMajorB;
    int boxesA, boxesB;             // TMA boxes per stage
    int chunkedA, chunkedB;         // the MN-major operand has a 4-d map: all its boxes of a stage arrive with one instruction
    int boxBytesA, boxBytesB;
    int boxElemsA, boxElemsB;       // elements of m / n per box when MN-major
    int batchMulA, batchMulB;       // 0: the operand is shared by every batch entry
    // Pointer-array batches: the matrices of entry e have their own tensor maps, entryMaps[3 e] (A), [3 e + 1] (B) and
    // [3 e + 2] (D), written to device memory by buildEntryMaps just before this launch; *entryFlag is non-zero when an
    // entry's pointers cannot be served by TMA, in which case this launch does nothing and the CUDA-core kernel behind it
    // does the work.
    const CUtensorMap* entryMaps;
    const unsigned* entryFlag;
    unsigned entrySerial;           // *entryFlag == entrySerial: stand down (the word needs no clearing between launches)
    int serpentine;                 // alternate units of a CTA walk the k slices in opposite directions
    int tmaStore;                   // D is 16-byte aligned in every dimension: results leave through shared memory and TMA
    int mirrorCount;                // every bulk store of D is repeated into this many other buffers (peer GPUs)
    // Split along k: a unit of work is (tile, split); the splits of a tile run on different CTAs at the same time, each
    // over its share of the k slices. All but the last to finish leave their accumulator in scratch memory; the last adds
    // them to its own, in split order, and writes D.
    int splits;                     // 1: no split
    long long totalUnits;           // totalTiles * splits
    unsigned* splitCounters;        // arrivals per half-tile slot; all zero between launches
    unsigned* splitPartials;        // [slot][split][column / 4][row][4] 32-bit accumulators
    EpilogueArgs epi;
};

// ---- PTX wrappers -----------------------------------------------------------------------------------------------

__device__ __forceinline__ unsigned smemAddr(const void* p) { return unsigned(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbarInit(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarArriveExpectTx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarArrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbarTryWait(unsigned bar, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
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

// Waits for the phase with `parity` to complete. Returns false when the CTA is aborting or the wait ran out
// of time; in the latter case the code is recorded and the abort flag raised for the other roles.
// SLEEP_NS > 0 puts the waiting thread to sleep between polls: the epilogue warps wait for most of a tile's main loop
// and share their scheduler with the warp that issues the MMAs, whose issue slots a polling loop would take.
template <unsigned SLEEP_NS>
__device__ __noinline__ bool mbarWaitSlow(unsigned bar, unsigned parity, volatile int* abortFlag, unsigned code) {
    const unsigned long long start = globalTimerNs();
    for (unsigned spins = 0;; ++spins) {
        if (mbarTryWait(bar, parity)) return true;
        if constexpr (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
        if ((spins & 63u) == 63u) {
            if (*abortFlag) return false;
            if (globalTimerNs() - start > kWaitLimitNs) {
                atomicCAS(&g_ummaStatus, kStatusOk, code);
                *abortFlag = 1;
                __threadfence_block();
                return false;
            }
        }
    }
}
template <unsigned SLEEP_NS = 0>
__device__ __forceinline__ bool mbarWait(unsigned bar, unsigned parity, volatile int* abortFlag, unsigned code) {
    if (mbarTryWait(bar, parity)) return true;
    return mbarWaitSlow<SLEEP_NS>(bar, parity, abortFlag, code);
}

// A tensor map that a kernel wrote to global memory is read through the tensor-map proxy only after this fence.
__device__ __forceinline__ void tensorMapAcquire(const CUtensorMap* map) {
    asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(reinterpret_cast<unsigned long long>(map)) : "memory");
}

__device__ __forceinline__ void tmaLoad3d(unsigned dst, const CUtensorMap* map, unsigned bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<unsigned long long>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// Shared memory -> global, asynchronous; elements outside the tensor are clipped by the hardware. The destination may be
// this GPU's memory or a peer's (the copy then travels over NVLink).
__device__ __forceinline__ void tmaStore3dIssue(const CUtensorMap* map, unsigned src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(reinterpret_cast<unsigned long long>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void tmaStoreCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Until at most `Pending` of this thread's bulk stores are still reading their shared-memory source.
template <int Pending>
__device__ __forceinline__ void tmaStoreWaitRead() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(Pending) : "memory");
}
__device__ __forceinline__ void tmaStoreWaitAll() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Barrier among the four warps of one epilogue group (hardware barriers 1 and 2; 0 is __syncthreads).
__device__ __forceinline__ void epilogueBarrier(int group) { asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory"); }

// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool electOne() {
    unsigned elected;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(elected));
    return elected != 0;
}

__device__ __forceinline__ void tcgen05FenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05FenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tcgen05Commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// One tcgen05.mma with kind and CTA group fixed at compile time: the issuing lane runs nothing but address arithmetic
// between two of these, and how fast it can issue them bounds the whole kernel (one MMA of 128 x 256 x 16 is 128 clocks of
// tensor-core work; every instruction the lane spends per MMA beyond that budget leaves the tensor cores idle).
template <int KIND, bool PAIR>
__device__ __forceinline__ void ummaIssueFixed(unsigned tmemD, unsigned long long descA, unsigned long long descB, unsigned idesc,
                                               unsigned accumulate) {
#define VKZB_UMMA(GROUP, KINDNAME)                                                                              \
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"                                              \
                 "tcgen05.mma.cta_group::" GROUP ".kind::" KINDNAME " [%0], %1, %2, %3, p;\n\t}"                   \
                 ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)                              \
                 : "memory")
    if constexpr (KIND == kKindF16) {
        if constexpr (PAIR) VKZB_UMMA("2", "f16"); else VKZB_UMMA("1", "f16");
    } else if constexpr (KIND == kKindI8) {
        if constexpr (PAIR) VKZB_UMMA("2", "i8"); else VKZB_UMMA("1", "i8");
    } else {
        if constexpr (PAIR) VKZB_UMMA("2", "tf32"); else VKZB_UMMA("1", "tf32");
    }
#undef VKZB_UMMA
}

// ---- two-CTA pairs (cta_group::2): the two CTAs of a cluster share one MMA of 256 rows ------------------------------

__device__ __forceinline__ unsigned clusterCtaRank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The shared::cluster address of the same shared-memory offset in the CTA of rank `rank`.
__device__ __forceinline__ unsigned mapToCta(unsigned localAddr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(localAddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void clusterSync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Load into this CTA's shared memory, completion counted on a barrier that may live in the pair's other CTA.
__device__ __forceinline__ void tmaLoad3dPair(unsigned dst, const CUtensorMap* map, unsigned clusterBar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<unsigned long long>(map)), "r"(clusterBar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// The same for a 4-d map (an operand contiguous along m or n, viewed as chunks of 128 bytes: see encodeChunked).
__device__ __forceinline__ void tmaLoad4d(unsigned dst, const CUtensorMap* map, unsigned bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<unsigned long long>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tmaLoad4dPair(unsigned dst, const CUtensorMap* map, unsigned clusterBar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<unsigned long long>(map)), "r"(clusterBar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// Arrives on the barrier at this offset in both CTAs of the pair once the MMAs issued so far have completed.
__device__ __forceinline__ void tcgen05CommitPair(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((unsigned short)3)
                 : "memory");
}
__device__ __forceinline__ void mbarArriveCluster(unsigned clusterBar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterBar) : "memory");
}
// 32 lanes x 32 columns of 32-bit accumulators: thread i of the warp receives row i, columns c .. c + 31.
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

// 32 columns without the wait: the values may be used only after tmemWaitLoads().
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
// The reverse of a 16-column load: thread i of the warp writes row i, columns c .. c + 15; complete when it returns.
__device__ __forceinline__ void tmemStore16(unsigned taddr, const unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// The same load without the wait: the values may be used only after tmemWaitLoads().
__device__ __forceinline__ void tmemLoad16Issue(unsigned taddr, unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
template <typename Acc>
__device__ __forceinline__ Acc accumulatorValue(unsigned bits) {
    if constexpr (std::is_same_v<Acc, int>) return int(bits);
    else return __uint_as_float(bits);
}

// 32 results of one row, consecutive columns, with the store form fixed at compile time. The addresses advance
// by one leading dimension per column, so each result costs an add, a multiply (plus a load and a fused
// multiply-add when beta != 0) and a store. `count` < 32 only in a tile's last, ragged chunk.
template <int MODE, typename Acc>
__device__ __forceinline__ void storeChunk(const Epilogue<Acc>& epi, const unsigned (&v)[32], int row, int col, int count) {
    using Elem = std::conditional_t<MODE == kStoreF32, float, std::conditional_t<MODE == kStoreS32, int,
                 std::conditional_t<MODE == kStoreF16, __half, __nv_bfloat16>>>;
    Elem* d = reinterpret_cast<Elem*>(epi.D) + (row + col * epi.ldd);
    const Elem* c = reinterpret_cast<const Elem*>(epi.C) + (row + col * epi.ldc);
    const Acc alpha = epi.alpha, beta = epi.beta;
    const long long ldd = epi.ldd, ldc = epi.ldc;
    const bool readC = epi.readC;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        if (j < count) {
            Acc r = alpha * accumulatorValue<Acc>(v[j]);
            if (readC) {
                if constexpr (MODE == kStoreF32 || MODE == kStoreS32) r += beta * Acc(*c);
                else if constexpr (MODE == kStoreF16) r += beta * __half2float(*c);
                else r += beta * __bfloat162float(*c);
                c += ldc;
            }
            if constexpr (MODE == kStoreF32 || MODE == kStoreS32) *d = r;
            else if constexpr (MODE == kStoreF16) *d = __float2half_rn(r);
            else *d = __float2bfloat16_rn(r);
            d += ldd;
        }
    }
}

// One accumulator (this warp's 32 rows; its group's share of the BN columns) from TMEM straight to global memory, 32 columns at
// a time, with the store form fixed at compile time. Out of line, one instance per form: the direct path serves the shapes
// TMA cannot (D not 16-byte aligned in every dimension), and keeping it out of the kernel body keeps the staged path lean.
template <int BN, int MODE, typename Acc>
__device__ __noinline__ void drainAccumulatorDirect(const Epilogue<Acc>& epi, unsigned taddr, int row, bool rowOk, int col0, int n, int group) {
#pragma unroll 1
    for (int c = group * 32; c < BN; c += 32 * kEpilogueGroups) {
        const int count = n - (col0 + c);
        if (count <= 0) break;
        unsigned v[32];
        tmemLoad32(taddr + c, v);
        if (!rowOk) continue;
        if constexpr (MODE == kStoreSlow) {
#pragma unroll 1
            for (int j = 0; j < 32; ++j) {
                unsigned bits = v[0];  // select v[j] without indexing registers dynamically
#pragma unroll
                for (int q = 1; q < 32; ++q) bits = j == q ? v[q] : bits;
                if (j < count) epi.storeSlow(row, col0 + c + j, accumulatorValue<Acc>(bits));
            }
        } else {
            storeChunk<MODE>(epi, v, row, col0 + c, count);
        }
    }
}

template <int BN, typename Acc>
__device__ __forceinline__ void drainAccumulator(const Epilogue<Acc>& epi, unsigned taddr, int row, bool rowOk, int col0, int n, int group) {
    if constexpr (std::is_same_v<Acc, int>) {
        if (epi.mode == kStoreS32) drainAccumulatorDirect<BN, kStoreS32>(epi, taddr, row, rowOk, col0, n, group);
        else drainAccumulatorDirect<BN, kStoreSlow>(epi, taddr, row, rowOk, col0, n, group);
    } else {
        if (epi.mode == kStoreF32) drainAccumulatorDirect<BN, kStoreF32>(epi, taddr, row, rowOk, col0, n, group);
        else if (epi.mode == kStoreF16) drainAccumulatorDirect<BN, kStoreF16>(epi, taddr, row, rowOk, col0, n, group);
        else if (epi.mode == kStoreBF16) drainAccumulatorDirect<BN, kStoreBF16>(epi, taddr, row, rowOk, col0, n, group);
        else drainAccumulatorDirect<BN, kStoreSlow>(epi, taddr, row, rowOk, col0, n, group);
    }
}

// The same through shared memory: each step's 128 x COLS block is laid out like the column-major D tile it belongs to
// (column pitch 128 elements; lane = row, so the writes are conflict-free), then one thread hands it to TMA, which
// writes full lines, clips rows and columns outside D, and keeps many stores in flight where four warps of scalar
// stores cannot. The NB buffers of a group take turns: a buffer is rewritten only after the bulk store that read it NB
// steps earlier has finished reading.
// One staged step: COLS columns of this warp's rows, already in registers, through a shared-memory buffer to a bulk store.
template <int MODE, int NB, int COLS, typename Acc>
__device__ __forceinline__ void stageAndStore(const Epilogue<Acc>& epi, const unsigned (&v)[COLS], int rowInTile, int row, bool rowOk,
                                              int row0, int col, int count, int batchEntry, const CUtensorMap* mapD, const MirrorMaps* mirrors,
                                              int mirrorCount, unsigned char* staging, unsigned& step, bool issuer, int group) {
    using Elem = std::conditional_t<MODE == kStoreF32, float, std::conditional_t<MODE == kStoreS32, int,
                 std::conditional_t<MODE == kStoreF16, __half, __nv_bfloat16>>>;
    const Acc alpha = epi.alpha, beta = epi.beta;
    Elem* buf = reinterpret_cast<Elem*>(staging + (step % NB + NB * group) * (kBM * COLS * 4)) + rowInTile;
    if constexpr (NB < 3) {  // two buffers: the one about to be rewritten is checked right here, and announced by a barrier
        if (issuer) tmaStoreWaitRead<1>();
        epilogueBarrier(group);
    }
    {
        if (epi.readC && rowOk) {
            const Elem* cin = reinterpret_cast<const Elem*>(epi.C) + (row + col * epi.ldc);
#pragma unroll
            for (int j = 0; j < COLS; ++j) {
                Acc r = alpha * accumulatorValue<Acc>(v[j]);
                if (j < count) {
                    if constexpr (MODE == kStoreF32 || MODE == kStoreS32) r += beta * Acc(cin[j * epi.ldc]);
                    else if constexpr (MODE == kStoreF16) r += beta * __half2float(cin[j * epi.ldc]);
                    else r += beta * __bfloat162float(cin[j * epi.ldc]);
                }
                if constexpr (MODE == kStoreF32 || MODE == kStoreS32) buf[j * kBM] = r;
                else if constexpr (MODE == kStoreF16) buf[j * kBM] = __float2half_rn(r);
                else buf[j * kBM] = __float2bfloat16_rn(r);
            }
        } else {
#pragma unroll
            for (int j = 0; j < COLS; ++j) {
                const Acc r = alpha * accumulatorValue<Acc>(v[j]);
                if constexpr (MODE == kStoreF32 || MODE == kStoreS32) buf[j * kBM] = r;
                else if constexpr (MODE == kStoreF16) buf[j * kBM] = __float2half_rn(r);
                else buf[j * kBM] = __float2bfloat16_rn(r);
            }
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    epilogueBarrier(group);
    if (issuer) {
        const unsigned src = smemAddr(buf - rowInTile);
        tmaStore3dIssue(mapD, src, row0, col, batchEntry);
        for (int q = 0; q < mirrorCount; ++q) tmaStore3dIssue(&mirrors->map[q], src, row0, col, batchEntry);  // the same block to every peer
        tmaStoreCommit();
        // more buffers: after this step's store is on its way, make sure the buffer of the step AFTER the next one is
        // free; the other warps learn it at the next step's barrier, before they reach that buffer
        if constexpr (NB >= 3) tmaStoreWaitRead<NB - 2>();
    }
    ++step;
}

// COLS columns of this lane's row: the sum over all splits in split order, `own` standing in for this CTA's split.
// `first` holds the same columns of split `firstOther` (the lowest split that is not this CTA's), loaded by the caller
// while it waited for TMEM; further splits are fetched here.
template <typename Acc, int COLS>
__device__ __forceinline__ void splitSum(unsigned (&own)[COLS], const uint4 (&first)[COLS / 4], int firstOther, const uint4* slotBase, size_t tileV4,
                                         int col, int splits, int split) {
    Acc sum[COLS];
#pragma unroll
    for (int j = 0; j < COLS; ++j) sum[j] = Acc(0);
#pragma unroll 1
    for (int s = 0; s < splits; ++s) {
        if (s == split) {
#pragma unroll
            for (int j = 0; j < COLS; ++j) sum[j] += accumulatorValue<Acc>(own[j]);
        } else {
            uint4 t[COLS / 4];
#pragma unroll
            for (int q = 0; q < COLS / 4; ++q) t[q] = s == firstOther ? first[q] : __ldcg(slotBase + size_t(s) * tileV4 + size_t(col / 4 + q) * kBM);
#pragma unroll
            for (int q = 0; q < COLS / 4; ++q) {
                sum[4 * q] += accumulatorValue<Acc>(t[q].x), sum[4 * q + 1] += accumulatorValue<Acc>(t[q].y);
                sum[4 * q + 2] += accumulatorValue<Acc>(t[q].z), sum[4 * q + 3] += accumulatorValue<Acc>(t[q].w);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < COLS; ++j) {
        if constexpr (std::is_same_v<Acc, int>) own[j] = unsigned(sum[j]);
        else own[j] = __float_as_uint(sum[j]);
    }
}

// The accumulator in staged steps of 32 columns (one TMEM load, one barrier, one fence and one bulk store per step). Measured on
// 256 x [1024 x 1024 x 128] with fp32 D, where the launch is bound by writing D: 16-column steps through 6 buffers per group
// took 287 us, 32 x 3 243 us, 32 x 4 223 us (16 x 6 with the next TMEM load in flight during a step: 272 us). The kernels for
// long k use two buffers per group and keep the shared memory for ring stages; with 32 columns per step they also stay
// within their registers (the 16-column form, two loads per wait, spilled 700 bytes).
constexpr int kStepCols = 32, kWideBuffers = 4;
template <int BN, int MODE, int NB, typename Acc>
__device__ __forceinline__ void drainAccumulatorStaged(const Epilogue<Acc>& epi, unsigned taddr, int rowInTile, int row, bool rowOk, int row0,
                                                           int col0, int n, int batchEntry, const CUtensorMap* mapD, const MirrorMaps* mirrors,
                                                           int mirrorCount, unsigned char* staging, unsigned& step, bool issuer, int group) {
#pragma unroll 1
    for (int c = group * kStepCols; c < BN; c += kStepCols * kEpilogueGroups) {
        const int count = n - (col0 + c);
        if (count <= 0) break;
        unsigned v[kStepCols];
        tmemLoad32Issue(taddr + c, v);
        tmemWaitLoads();
        stageAndStore<MODE, NB, kStepCols>(epi, v, rowInTile, row, rowOk, row0, col0 + c, count, batchEntry, mapD, mirrors, mirrorCount, staging,
                                                         step, issuer, group);
    }
}

// The same after a split along k, by the split that writes D: the other splits' accumulators (splitBase: this lane's row in
// the tile's scratch slot) are added on the way, their first loads travelling while TMEM delivers. Out of line, so that its
// registers are not the main path's.
template <int BN, int MODE, int NB, typename Acc>
__device__ __noinline__ void drainAccumulatorStagedSplit(const Epilogue<Acc>& epi, unsigned taddr, int rowInTile, int row, bool rowOk, int row0,
                                                         int col0, int n, int batchEntry, const CUtensorMap* mapD, unsigned char* staging,
                                                         unsigned& step, bool issuer, int group, const uint4* splitBase, int splits, int split) {
    const size_t tileV4 = size_t(BN) * kBM / 4;
    const int firstOther = split == 0 ? 1 : 0;
#pragma unroll 1
    for (int c = group * kStepCols; c < BN; c += kStepCols * kEpilogueGroups) {
        const int count = n - (col0 + c);
        if (count <= 0) break;
        unsigned v[kStepCols];
        uint4 first[kStepCols / 4];
        tmemLoad32Issue(taddr + c, v);
#pragma unroll
        for (int q = 0; q < kStepCols / 4; ++q) first[q] = __ldcg(splitBase + size_t(firstOther) * tileV4 + size_t(c / 4 + q) * kBM);
        tmemWaitLoads();
        splitSum<Acc, kStepCols>(v, first, firstOther, splitBase, tileV4, c, splits, split);
        stageAndStore<MODE, NB, kStepCols>(epi, v, rowInTile, row, rowOk, row0, col0 + c, count, batchEntry, mapD, nullptr, 0, staging, step, issuer, group);
    }
}

// The same with a bias vector, an activation or the extra rounding after alpha * acc + beta * C (cublasLtMatmul epilogues): the
// finished values go through the staged store as they are (alpha 1, no C). Out of line like the split form.
template <int BN, int MODE, int NB>
__device__ __noinline__ void drainAccumulatorStagedPost(const Epilogue<float>& epi, unsigned taddr, int rowInTile, int row, bool rowOk, int row0,
                                                        int col0, int n, int batchEntry, const CUtensorMap* mapD, const MirrorMaps* mirrors,
                                                        int mirrorCount, unsigned char* staging, unsigned& step, bool issuer, int group) {
    using Elem = std::conditional_t<MODE == kStoreF32, float, std::conditional_t<MODE == kStoreF16, __half, __nv_bfloat16>>;
    Epilogue<float> plain = epi;
    plain.alpha = 1.0f, plain.readC = false;
    const float rowBias = epi.bias && rowOk && !epi.biasAlongN ? loadAs<float>(epi.bias, row, epi.typeBias) : 0.0f;
    const bool colBias = epi.bias && epi.biasAlongN;
    const int lane = threadIdx.x % 32;
#pragma unroll 1
    for (int c = group * kStepCols; c < BN; c += kStepCols * kEpilogueGroups) {
        const int count = n - (col0 + c);
        if (count <= 0) break;
        unsigned v[kStepCols];
        tmemLoad32Issue(taddr + c, v);
        tmemWaitLoads();
        const Elem* cin = reinterpret_cast<const Elem*>(epi.C) + (row + (long long)(col0 + c) * epi.ldc);
#pragma unroll
        for (int j = 0; j < kStepCols; ++j) {
            float r = epi.alpha * __uint_as_float(v[j]);
            if (epi.readC && rowOk && j < count) {
                if constexpr (MODE == kStoreF32) r += epi.beta * cin[j * epi.ldc];
                else if constexpr (MODE == kStoreF16) r += epi.beta * __half2float(cin[j * epi.ldc]);
                else r += epi.beta * __bfloat162float(cin[j * epi.ldc]);
            }
            const float biasValue = colBias && j < count ? loadAs<float>(epi.bias, col0 + c + j, epi.typeBias) : rowBias;
            if (!epi.aux) {
                v[j] = __float_as_uint(epi.finish(r, biasValue));
                continue;
            }
            // with an auxiliary matrix: a warp holds 32 consecutive rows of one column, so a ReLU mask leaves (and arrives)
            // as one 32-bit word per warp and column, a GELU input as one 128-byte (or 64-byte) line
            if (epi.roundBeforeBias) r = roundTo(r, epi.typeD);
            r += biasValue;
            const long long at = row + (long long)(col0 + c + j) * epi.auxLd;  // row - lane is a multiple of 32, and so is auxLd for masks
            const bool live = j < count;
            if (epi.auxMode == kAuxWriteMask) {
                const unsigned word = __ballot_sync(0xFFFFFFFFu, rowOk && r > 0.0f);
                if (lane == 0 && live) reinterpret_cast<unsigned*>(epi.aux)[at >> 5] = word;
            } else if (epi.auxMode == kAuxWriteInput) {
                if (rowOk && live) storeFloat(epi.aux, at, epi.typeAux, r);
            }
            if (epi.activation == kActRelu) r = fmaxf(r, 0.0f);
            else if (epi.activation == kActGelu) r = geluTanh(r);
            else if (epi.activation == kActDRelu) r = live && ((reinterpret_cast<const unsigned*>(epi.aux)[(at - lane) >> 5] >> lane) & 1u) ? r : 0.0f;
            else if (epi.activation == kActDGelu) r = rowOk && live ? r * geluTanhGrad(loadAs<float>(epi.aux, at, epi.typeAux)) : 0.0f;
            v[j] = __float_as_uint(r);
        }
        stageAndStore<MODE, NB, kStepCols>(plain, v, rowInTile, row, rowOk, row0, col0 + c, count, batchEntry, mapD, mirrors, mirrorCount, staging, step, issuer,
                                           group);
    }
}

// Barrier among all eight epilogue warps (hardware barrier 3).
__device__ __forceinline__ void epilogueBarrierAll() { asm volatile("bar.sync 3, %0;" ::"n"(32 * kEpilogueWarps) : "memory"); }

// The hand-over between the splits of a tile. Scratch memory holds, per half-tile slot and split, this CTA's 128 rows by BN
// columns of 32-bit accumulators as 16-byte groups of 4 columns, lane = row: group (column / 4) of row r is uint4 number
// (column / 4) * 128 + r, so a warp moves 512 contiguous bytes per access.
//
// splitDump, run by all epilogue warps once this CTA's accumulator is complete: write the accumulator to this split's place
// and count the split in. Returns true in the split that finds all others counted already: that one sums the accumulators
// in split order (its own from TMEM: the order of the additions does not depend on who came last, so the result is the same
// from run to run) and writes D. The others are done with the tile. Nobody waits for anybody.
template <int BN>
__device__ __noinline__ bool splitDump(unsigned* counters, unsigned* partials, int splits, unsigned taddr, long long slot, int split, int quarter,
                                       int lane, int group, volatile int* lastFlag) {
    constexpr int kStride = kStoreCols * kEpilogueGroups, kSteps = BN / kStride, kBatch = kSteps < 4 ? kSteps : 4;
    uint4* mine = reinterpret_cast<uint4*>(partials + (size_t(slot) * splits + split) * (size_t(BN) * kBM)) + quarter * 32 + lane;
#pragma unroll 1
    for (int c = group * kStoreCols; c < BN; c += kBatch * kStride) {
        unsigned v[kBatch][kStoreCols];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) tmemLoad16Issue(taddr + c + b * kStride, v[b]);
        tmemWaitLoads();
#pragma unroll
        for (int b = 0; b < kBatch; ++b)
#pragma unroll
            for (int q = 0; q < 4; ++q)
                __stcg(mine + size_t((c + b * kStride) / 4 + q) * kBM, make_uint4(v[b][4 * q], v[b][4 * q + 1], v[b][4 * q + 2], v[b][4 * q + 3]));
    }
    __threadfence();
    epilogueBarrierAll();
    if (threadIdx.x == 64) {
        const unsigned before = atomicAdd(counters + slot, 1u);
        const bool last = before == unsigned(splits - 1);
        if (last) counters[slot] = 0;  // every split has arrived: ready for the next launch
        __threadfence();
        *lastFlag = last;
    }
    epilogueBarrierAll();
    return *lastFlag != 0;
}

// For the store paths that read TMEM themselves (direct stores): the last split puts the sum back into TMEM first.
template <int BN, typename Acc>
__device__ __noinline__ void splitSumToTmem(const unsigned* partials, int splits, unsigned taddr, long long slot, int split, int quarter, int lane,
                                            int group) {
    const size_t tileV4 = size_t(BN) * kBM / 4;
    const uint4* slotBase = reinterpret_cast<const uint4*>(partials) + size_t(slot) * splits * tileV4 + quarter * 32 + lane;
    const int firstOther = split == 0 ? 1 : 0;
#pragma unroll 1
    for (int c = group * kStoreCols; c < BN; c += kStoreCols * kEpilogueGroups) {
        unsigned own[kStoreCols];
        uint4 first[4];
        tmemLoad16Issue(taddr + c, own);
#pragma unroll
        for (int q = 0; q < 4; ++q) first[q] = __ldcg(slotBase + size_t(firstOther) * tileV4 + size_t(c / 4 + q) * kBM);
        tmemWaitLoads();
        splitSum<Acc, kStoreCols>(own, first, firstOther, slotBase, tileV4, c, splits, split);
        tmemStore16(taddr + c, own);
    }
    // the store paths divide the columns between the groups differently: both groups' sums are in TMEM before either reads
    tcgen05FenceBefore();
    epilogueBarrierAll();
    tcgen05FenceAfter();
}

// Tile number -> (batch entry, tile row, tile column). Tiles are numbered so that consecutive numbers, which run
// at the same time on neighbouring SMs, cover `groupM` tile rows by a few tile columns: their A and B panels
// are then fetched from HBM once and served from L2 to the other CTAs that need them.
struct TileCoord {
    int batch, row, col;
};
__device__ __forceinline__ TileCoord tileCoord(const UmmaArgs& g, long long tile) {
    const int perEntry = g.tilesM * g.tilesN;
    const int batch = int(tile / perEntry), r = int(tile % perEntry);
    const int groupSize = g.groupM * g.tilesN;
    const int group = r / groupSize, firstRow = group * g.groupM;
    const int rowsInGroup = min(g.tilesM - firstRow, g.groupM);
    const int inGroup = r % groupSize;
    return {batch, firstRow + inGroup % rowsInGroup, inGroup / rowsInGroup};
}

// PAIR: the kernel runs as clusters of two CTAs that share each MMA (M = 256): a CTA stages its own 128 rows of A and only
// half of the tile's B columns, so a k slice costs it (128 + BN / 2) rows of 128 bytes from L2 instead of (128 + BN).
// WIDE: for products with few k slices per tile the time goes into writing D, not into the main loop. Such launches
// trade ring stages for epilogue buffers: 64 KiB of staging buffers per warp group instead of 16 KiB keep enough bulk stores
// in flight to cover the latency of a store, and the steps are 32 columns wide (drainAccumulatorStaged).
template <int BN, bool PAIR, bool WIDE>
struct SmemPlan {
    static constexpr int kCtaB = PAIR ? BN / 2 : BN;  // B rows (tile columns) this CTA stages
    static constexpr int kStageBBytes = kCtaB * kSliceBytes;
    static constexpr int kStageBytes = kStageABytes + kStageBBytes;
    static constexpr int kStagingBuffers = WIDE ? 2 * kWideBuffers : 4;  // per epilogue group, in units of 8 KiB: four or two steps of 32 columns
    static constexpr int kStagingBytes = kEpilogueGroups * kStagingBuffers * kStagingBufferBytes;
    static constexpr int kOverhead = 1024 /* alignment slack */ + 256 /* barriers */;
    static constexpr int kStages = (kSmemTotal - kStagingBytes - kOverhead) / kStageBytes > 12 ? 12 : (kSmemTotal - kStagingBytes - kOverhead) / kStageBytes;
    static constexpr int kTmemCols = 2 * BN;  // two accumulators of BN columns for this CTA's 128 rows
    static constexpr int kDynamicBytes = kStages * kStageBytes + kStagingBytes + kOverhead;
    static_assert(kStages >= 2, "ring length");
    static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols >= 32 && kTmemCols <= 512, "TMEM allocation size");
    static_assert(kDynamicBytes <= kSmemTotal, "shared memory");
};

// The TMA producer's loop. KMAJOR: both operands are contiguous along k (op(A) = A^T, op(B) = B), one box each per stage;
// otherwise an operand that is contiguous along m or n arrives as several boxes of 128 bytes by slice-length rows.
template <int BN, bool PAIR, bool WIDE, bool KMAJOR>
__device__ __forceinline__ void producerLoop(const UmmaArgs& g, const CUtensorMap* launchMapA, const CUtensorMap* launchMapB, unsigned smemBase,
                                             unsigned fullBar, unsigned emptyBar, unsigned ctaRank, long long firstUnit, long long unitStride,
                                             volatile int* abortFlag) {
    using Plan = SmemPlan<BN, PAIR, WIDE>;
    constexpr int kStages = Plan::kStages;
    constexpr int kTileRows = PAIR ? 2 * kBM : kBM;
    const bool leader = ctaRank == 0;
    // completion of both CTAs' loads is counted on the leader's barrier, where the MMA issuer waits
    const unsigned fullBarLeader = PAIR ? mapToCta(fullBar, 0) : fullBar;
    const int slices = g.numKSlices, sliceElems = g.sliceElems;
    int stage = 0;
    unsigned phase = 0;
    bool backwards = false;
    for (long long unit = firstUnit; unit < g.totalUnits; unit += unitStride, backwards = !backwards) {
        const int split = int(unit % g.splits);
        const TileCoord t = tileCoord(g, unit / g.splits);
        const int row0 = t.row * kTileRows + int(ctaRank) * kBM, col0 = t.col * BN + int(ctaRank) * Plan::kCtaB;
        // a pointer-array batch: this entry's own maps (batch coordinate 0), made by the kernel before this one
        const CUtensorMap* mapA = g.entryMaps ? g.entryMaps + 3 * t.batch : launchMapA;
        const CUtensorMap* mapB = g.entryMaps ? g.entryMaps + 3 * t.batch + 1 : launchMapB;
        if (g.entryMaps) tensorMapAcquire(mapA), tensorMapAcquire(mapB);
        const int batchA = g.entryMaps ? 0 : t.batch * g.batchMulA, batchB = g.entryMaps ? 0 : t.batch * g.batchMulB;
        // Every other unit of a CTA walks k from the far end: the CTAs of a wave move along k together, so the slices they all
        // used last are the ones the next wave's tiles in the same rows find in L2 first.
        const int ksFirst = int((long long)slices * split / g.splits), ksEnd = int((long long)slices * (split + 1) / g.splits);
        for (int step = ksFirst; step < ksEnd; ++step) {
            const int ks = g.serpentine && backwards ? ksEnd - 1 - (step - ksFirst) : step;
            if (!mbarWait(emptyBar + 8 * stage, phase ^ 1, abortFlag, kStatusProducerWait)) return;
            const unsigned bar = fullBarLeader + 8 * stage;
            if (leader) mbarArriveExpectTx(fullBar + 8 * stage, unsigned(Plan::kStageBytes) * (PAIR ? 2u : 1u));
            const unsigned dstA = smemBase + stage * Plan::kStageBytes, dstB = dstA + kStageABytes;
            const int k0 = ks * sliceElems;
            const auto load = [&](unsigned dst, const CUtensorMap* map, int c0, int c1, int c2) {
                if constexpr (PAIR) tmaLoad3dPair(dst, map, bar, c0, c1, c2);
                else tmaLoad3d(dst, map, bar, c0, c1, c2);
            };
            if constexpr (KMAJOR) {
                load(dstA, mapA, k0, row0, batchA);
                load(dstB, mapB, k0, col0, batchB);
            } else {
                const auto loadChunks = [&](unsigned dst, const CUtensorMap* map, int mn0, int elems, int batchEntry) {
                    if constexpr (PAIR) tmaLoad4dPair(dst, map, bar, 0, k0, mn0 / elems, batchEntry);
                    else tmaLoad4d(dst, map, bar, 0, k0, mn0 / elems, batchEntry);
                };
                if (g.chunkedA) {
                    loadChunks(dstA, mapA, row0, g.boxElemsA, batchA);
                } else if (g.mnMajorA) {
                    for (int b = 0; b < g.boxesA; ++b) load(dstA + b * g.boxBytesA, mapA, row0 + b * g.boxElemsA, k0, batchA);
                } else {
                    load(dstA, mapA, k0, row0, batchA);
                }
                if (g.chunkedB) {
                    loadChunks(dstB, mapB, col0, g.boxElemsB, batchB);
                } else if (g.mnMajorB) {
                    for (int b = 0; b < g.boxesB; ++b) load(dstB + b * g.boxBytesB, mapB, col0 + b * g.boxElemsB, k0, batchB);
                } else {
                    load(dstB, mapB, k0, col0, batchB);
                }
            }
            if (++stage == kStages) stage = 0, phase ^= 1;
        }
    }
}

// The MMA issuer's loop for one operand kind. The whole warp walks it (so addresses and descriptors are warp-uniform
// values), one elected lane issues. Per k slice: wait for the stage, four MMAs whose descriptors differ by a constant,
// one commit that frees the stage when they have read it.
template <int BN, bool PAIR, bool WIDE, int KIND>
__device__ __forceinline__ void mmaIssuerLoop(const UmmaArgs& g, unsigned smemBase, unsigned fullBar, unsigned emptyBar, unsigned accFullBar,
                                              unsigned accEmptyBar, unsigned tmemBase, long long firstUnit, long long unitStride,
                                              volatile int* abortFlag) {
    using Plan = SmemPlan<BN, PAIR, WIDE>;
    constexpr int kStages = Plan::kStages;
    const unsigned long long hi = static_cast<unsigned long long>(g.descHi) << 32;
    const unsigned lboA = g.lboA << 16, lboB = g.lboB << 16, stepA = g.kStepA, stepB = g.kStepB, idesc = g.idesc;
    const int slices = g.numKSlices;
    int stage = 0;
    unsigned phase = 0, tileCount = 0;
    bool ok = true;
    for (long long unit = firstUnit; ok && unit < g.totalUnits; unit += unitStride, ++tileCount) {
        const unsigned acc = tileCount & 1, accPhase = (tileCount >> 1) & 1;
        if (!(ok = mbarWait(accEmptyBar + 8 * acc, accPhase ^ 1, abortFlag, kStatusMmaTmemWait))) break;
        tcgen05FenceAfter();
        const unsigned tmemD = tmemBase + acc * BN;
        const int split = int(unit % g.splits);
        const int ksBegin = int((long long)slices * split / g.splits), ksEnd = int((long long)slices * (split + 1) / g.splits);
        for (int ks = ksBegin; ks < ksEnd; ++ks) {
            if (!(ok = mbarWait(fullBar + 8 * stage, phase, abortFlag, kStatusMmaFullWait))) break;
            tcgen05FenceAfter();
            const unsigned addrA = smemBase + stage * Plan::kStageBytes, addrB = addrA + kStageABytes;
            const unsigned long long descA = hi | (((addrA & 0x3FFFFu) >> 4) | lboA), descB = hi | (((addrB & 0x3FFFFu) >> 4) | lboB);
            if (electOne()) {
                ummaIssueFixed<KIND, PAIR>(tmemD, descA, descB, idesc, ks != ksBegin ? 1u : 0u);
#pragma unroll
                for (int j = 1; j < kMmasPerStage; ++j)  // the low word cannot carry into the high one: addresses stay below 2^14 units
                    ummaIssueFixed<KIND, PAIR>(tmemD, descA + j * stepA, descB + j * stepB, idesc, 1u);
                // the stage may be refilled (in both CTAs of a pair) once these MMAs have read it
                if constexpr (PAIR) tcgen05CommitPair(emptyBar + 8 * stage);
                else tcgen05Commit(emptyBar + 8 * stage);
            }
            __syncwarp();
            if (++stage == kStages) stage = 0, phase ^= 1;
        }
        if (ok && electOne()) {
            if constexpr (PAIR) tcgen05CommitPair(accFullBar + 8 * acc);
            else tcgen05Commit(accFullBar + 8 * acc);
        }
        __syncwarp();
    }
}

template <int BN, bool PAIR, bool WIDE>
__global__ void __launch_bounds__(kThreads, 1)
ummaGemmKernel(const UmmaArgs g, const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
               const __grid_constant__ CUtensorMap mapD, const __grid_constant__ MirrorMaps mirrors) {
    using Plan = SmemPlan<BN, PAIR, WIDE>;
    constexpr int kStages = Plan::kStages;
    if (g.entryFlag && *g.entryFlag == g.entrySerial) return;  // an entry of the pointer-array batch is not fit for TMA: every CTA leaves at once
    extern __shared__ unsigned char smemRaw[];
    // the swizzled layout is defined on 1024-byte aligned addresses
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
    unsigned char* staging = smem + kStages * Plan::kStageBytes;  // epilogue buffers, 1024-byte aligned like the stages
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(staging + Plan::kStagingBytes);
    // bars[0 .. S): stage filled; [S .. 2S): stage drained; [2S, 2S+2): accumulator ready; [2S+2, 2S+4): accumulator drained
    unsigned* tmemSlot = reinterpret_cast<unsigned*>(bars + 2 * kStages + 4);
    volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const unsigned smemBase = smemAddr(smem);
    const unsigned fullBar = smemAddr(bars), emptyBar = fullBar + 8 * kStages;
    const unsigned accFullBar = emptyBar + 8 * kStages, accEmptyBar = accFullBar + 16;
    // In a pair, CTA 0 (the leader) issues the MMAs for both; work is dealt to pairs, not CTAs.
    const unsigned ctaRank = PAIR ? clusterCtaRank() : 0u;
    const bool leader = ctaRank == 0;
    const long long firstUnit = PAIR ? blockIdx.x / 2 : blockIdx.x, unitStride = PAIR ? gridDim.x / 2 : gridDim.x;
    constexpr int kTileRows = PAIR ? 2 * kBM : kBM;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbarInit(fullBar + 8 * s, 1);
            mbarInit(emptyBar + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbarInit(accFullBar + 8 * a, 1);
            mbarInit(accEmptyBar + 8 * a, kEpilogueWarps * (PAIR ? 2 : 1));  // the leader hears from both CTAs' epilogues
        }
        *abortFlag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        if constexpr (PAIR) {  // the same warp of both CTAs allocates the same columns in both TMEMs
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(tmemSlot)),
                         "r"(unsigned(Plan::kTmemCols))
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(tmemSlot)),
                         "r"(unsigned(Plan::kTmemCols))
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tcgen05FenceBefore();
    __syncthreads();
    if constexpr (PAIR) clusterSync();  // the other CTA's barriers exist before anything is signalled on them
    tcgen05FenceAfter();
    const unsigned tmemBase = *tmemSlot;

    if (warp == 0) {
        // ---- TMA producer ----
        if (lane == 0) {
            if (!g.mnMajorA && !g.mnMajorB)
                producerLoop<BN, PAIR, WIDE, true>(g, &mapA, &mapB, smemBase, fullBar, emptyBar, ctaRank, firstUnit, unitStride, abortFlag);
            else
                producerLoop<BN, PAIR, WIDE, false>(g, &mapA, &mapB, smemBase, fullBar, emptyBar, ctaRank, firstUnit, unitStride, abortFlag);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---- MMA issuer (in a pair: the leader only) ----
        if (leader) {
            if (g.kind == kKindF16)
                mmaIssuerLoop<BN, PAIR, WIDE, kKindF16>(g, smemBase, fullBar, emptyBar, accFullBar, accEmptyBar, tmemBase, firstUnit, unitStride, abortFlag);
            else if (g.kind == kKindI8)
                mmaIssuerLoop<BN, PAIR, WIDE, kKindI8>(g, smemBase, fullBar, emptyBar, accFullBar, accEmptyBar, tmemBase, firstUnit, unitStride, abortFlag);
            else
                mmaIssuerLoop<BN, PAIR, WIDE, kKindTf32>(g, smemBase, fullBar, emptyBar, accFullBar, accEmptyBar, tmemBase, firstUnit, unitStride, abortFlag);
        }
        __syncwarp();
    } else {
        // ---- epilogue: TMEM -> registers -> global ----
        const int quarter = warp % 4;  // a warp may only touch TMEM lanes 32 * (warp % 4) .. + 31
        const int group = (warp - 2) / 4;
        unsigned tileCount = 0, storeStep = 0;
        const bool issuer = threadIdx.x == 64 + 128 * group;  // first lane of the group's first warp owns its bulk stores
        bool ok = true;
        for (long long unit = firstUnit; ok && unit < g.totalUnits; unit += unitStride, ++tileCount) {
            const long long tile = unit / g.splits;
            const TileCoord t = tileCoord(g, tile);
            const unsigned acc = tileCount & 1, accPhase = (tileCount >> 1) & 1;
            if (lane == 0) mbarWait(accFullBar + 8 * acc, accPhase, abortFlag, kStatusEpilogueWait);  // one poller per warp
            epilogueBarrier(group);  // the four warps take the same decision: a wait that gave up has raised the flag by now
            ok = *abortFlag == 0;
            if (!ok) break;
            tcgen05FenceAfter();
            const int tileRow0 = t.row * kTileRows + int(ctaRank) * kBM;  // this CTA's 128 rows of the tile
            const int row = tileRow0 + quarter * 32 + lane;
            const int col0 = t.col * BN;
            const unsigned taddr = tmemBase + acc * BN + (unsigned(quarter * 32) << 16);
            const bool rowOk = row < g.m;
            const int rowInTile = quarter * 32 + lane;
            const CUtensorMap* unitMapD = g.entryMaps ? g.entryMaps + 3 * t.batch + 2 : &mapD;
            const int storeEntry = g.entryMaps ? 0 : t.batch;  // the batch coordinate of the bulk stores
            if (g.entryMaps && issuer) tensorMapAcquire(unitMapD);
            // After a split along k: hand the accumulator over. True when this CTA goes on to write D; `splitBase` is then
            // set for the staged stores, which add the other splits' accumulators on their way, while for the direct
            // stores the sum has been put back into TMEM.
            const uint4* splitBase = nullptr;
            const int split = int(unit % g.splits);
            const auto handOver = [&](bool staged, auto accTag) {
                if (g.splits == 1) return true;
                const long long slot = PAIR ? tile * 2 + ctaRank : tile;
                if (!splitDump<BN>(g.splitCounters, g.splitPartials, g.splits, taddr, slot, split, quarter, lane, group, abortFlag + 1)) return false;
                if (staged) splitBase = reinterpret_cast<const uint4*>(g.splitPartials) + size_t(slot) * g.splits * (size_t(BN) * kBM / 4) + rowInTile;
                else splitSumToTmem<BN, decltype(accTag)>(g.splitPartials, g.splits, taddr, slot, split, quarter, lane, group);
                return true;
            };
            if (g.kind == kKindI8) {
                Epilogue<int> epi;
                epi.init(g.epi, t.batch);
                const bool staged = g.tmaStore && epi.mode == kStoreS32;
                if (!handOver(staged, int(0))) {
                    // another split of this tile writes D
                } else if (staged) {
                    if (splitBase) drainAccumulatorStagedSplit<BN, kStoreS32, 2>(epi, taddr, rowInTile, row, rowOk, tileRow0, col0, g.n, storeEntry, unitMapD, staging, storeStep, issuer, group, splitBase, g.splits, split);
                    else drainAccumulatorStaged<BN, kStoreS32, (WIDE ? kWideBuffers : 2)>(epi, taddr, rowInTile, row, rowOk, tileRow0, col0, g.n, storeEntry, unitMapD, &mirrors, g.mirrorCount, staging, storeStep, issuer, group);
                } else {
                    drainAccumulator<BN>(epi, taddr, row, rowOk, col0, g.n, group);
                }
            } else {
                Epilogue<float> epi;
                epi.init(g.epi, t.batch);
                const bool staged = g.tmaStore && epi.mode != kStoreSlow;
                // bias, activation, extra rounding: staged as well when C and D alone would be (after a split the sum goes back to TMEM first)
                const bool stagedPost = g.tmaStore && epi.post && epi.typedMode != kStoreSlow;
                constexpr int kBuffers = WIDE ? kWideBuffers : 2;
                if (!handOver(staged, float(0))) {
                    // another split of this tile writes D
                } else if (stagedPost && epi.typedMode == kStoreF32) {
                    drainAccumulatorStagedPost<BN, kStoreF32, kBuffers>(epi, taddr, rowInTile, row, rowOk, tileRow0, col0, g.n, storeEntry, unitMapD, &mirrors, g.mirrorCount, staging, storeStep, issuer, group);
                } else if (stagedPost && epi.typedMode == kStoreF16) {
                    drainAccumulatorStagedPost<BN, kStoreF16, kBuffers>(epi, taddr, rowInTile, row, rowOk, tileRow0, col0, g.n, storeEntry, unitMapD, &mirrors, g.mirrorCount, staging, storeStep, issuer, group);
                } else if (stagedPost && epi.typedMode == kStoreBF16) {
                    drainAccumulatorStagedPost<BN, kStoreBF16, kBuffers>(epi, taddr, rowInTile, row, rowOk, tileRow0, col0, g.n, storeEntry, unitMapD, &mirrors, g.mirrorCount, staging, storeStep, issuer, group);
                } else if (staged && epi.mode == kStoreF32) {
                    if (splitBase) drainAccumulatorStagedSplit<BN, kStoreF32, 2>(epi, taddr, rowInTile, row, rowOk, tileRow0, col0, g.n, storeEntry, unitMapD, staging, storeStep, issuer, group, splitBase, g.splits, split);
                    else drainAccumulatorStaged<BN, kStoreF32, (WIDE ? kWideBuffers : 2)>(epi, taddr, rowInTile, row, rowOk, tileRow0, col0, g.n, storeEntry, unitMapD, &mirrors, g.mirrorCount, staging, storeStep, issuer, group);
                } else if (staged && epi.mode == kStoreF16) {
                    if (splitBase) drainAccumulatorStagedSplit<BN, kStoreF16, 2>(epi, taddr, rowInTile, row, rowOk, tileRow0, col0, g.n, storeEntry, unitMapD, staging, storeStep, issuer, group, splitBase, g.splits, split);
                    else drainAccumulatorStaged<BN, kStoreF16, (WIDE ? kWideBuffers : 2)>(epi, taddr, rowInTile, row, rowOk, tileRow0, col0, g.n, storeEntry, unitMapD, &mirrors, g.mirrorCount, staging, storeStep, issuer, group);
                } else if (staged && epi.mode == kStoreBF16) {
                    if (splitBase) drainAccumulatorStagedSplit<BN, kStoreBF16, 2>(epi, taddr, rowInTile, row, rowOk, tileRow0, col0, g.n, storeEntry, unitMapD, staging, storeStep, issuer, group, splitBase, g.splits, split);
                    else drainAccumulatorStaged<BN, kStoreBF16, (WIDE ? kWideBuffers : 2)>(epi, taddr, rowInTile, row, rowOk, tileRow0, col0, g.n, storeEntry, unitMapD, &mirrors, g.mirrorCount, staging, storeStep, issuer, group);
                } else {
                    drainAccumulator<BN>(epi, taddr, row, rowOk, col0, g.n, group);
                }
            }
            tcgen05FenceBefore();
            __syncwarp();
            if (lane == 0) {
                if constexpr (PAIR) mbarArriveCluster(mapToCta(accEmptyBar + 8 * acc, 0));
                else mbarArrive(accEmptyBar + 8 * acc);
            }
        }
        if (issuer) tmaStoreWaitAll();  // the bulk stores read shared memory and must be done before the CTA ends
    }

    // ---- common exit ----
    if (*abortFlag) __nanosleep(20000);  // let copies still in flight land before the shared memory is released
    tcgen05FenceBefore();
    __syncthreads();
    if constexpr (PAIR) clusterSync();  // neither CTA leaves while the other may still read its shared memory or signal it
    if (warp == 1) {
        tcgen05FenceAfter();
        if constexpr (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(unsigned(Plan::kTmemCols)) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(unsigned(Plan::kTmemCols)) : "memory");
    }
}

// Pointer-array batches: one thread per batch entry copies the launch's template maps (right shape, strides and boxes, a
// placeholder address) to entryMaps[3 e ..] and puts the entry's own addresses in with tensormap.replace. An entry whose
// pointers TMA cannot take (not 16-byte aligned; D only when the launch stores D through TMA) writes the launch's serial
// number to the flag word instead.
__global__ void buildEntryMaps(const __grid_constant__ CUtensorMap templateA, const __grid_constant__ CUtensorMap templateB,
                               const __grid_constant__ CUtensorMap templateD, const void* const* A, const void* const* B, void* const* D, int batch,
                               int storeThroughTma, CUtensorMap* entryMaps, unsigned* flag, unsigned serial) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= batch) return;
    const unsigned long long a = reinterpret_cast<unsigned long long>(A[e]), b = reinterpret_cast<unsigned long long>(B[e]),
                             d = reinterpret_cast<unsigned long long>(D[e]);
    if ((a & 15) || (b & 15) || (storeThroughTma && (d & 15)) || !a || !b || !d) {
        *flag = serial;  // this launch's own number: nothing else ever writes it, so the word is never cleared
        return;
    }
    CUtensorMap* mine = entryMaps + 3 * e;
    mine[0] = templateA, mine[1] = templateB, mine[2] = templateD;
    __threadfence();
    const auto setAddress = [](CUtensorMap* map, unsigned long long address) {
        asm volatile("tensormap.replace.tile.global_address.global.b1024.b64 [%0], %1;" ::"l"(reinterpret_cast<unsigned long long>(map)), "l"(address) : "memory");
    };
    setAddress(mine, a), setAddress(mine + 1, b), setAddress(mine + 2, d);
    asm volatile("fence.proxy.tensormap::generic.release.gpu;" ::: "memory");
}

// ---- host side ---------------------------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encodeTiled() {
    static const EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

struct DeviceInfo {
    int sms = 0;
    bool sm100 = false;
    bool attrSet[10] = {};
    int clusters[10] = {};  // concurrent two-CTA clusters per kernel variant
};

DeviceInfo& deviceInfo() {
    static std::mutex mutex;
    static DeviceInfo info[64];
    int dev = 0;
    cudaGetDevice(&dev);
    dev = dev < 0 || dev >= 64 ? 0 : dev;
    std::lock_guard<std::mutex> lock(mutex);
    DeviceInfo& d = info[dev];
    if (!d.sms) {
        int major = 0;
        cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        d.sm100 = major == 10;
        if (d.sms <= 0) d.sms = 1;
    }
    return d;
}

int elemSizeOf(int type) { return type == kF32 ? 4 : type == kS8 ? 1 : 2; }

// How much L2 fetches around each line an operand load asks for.
CUtensorMapL2promotion operandPromotion() {
    static const int forced = measureKnob("VKZB_UMMA_L2_PROMOTION", 3);  // 0 none, 1 64 bytes, 2 128 bytes, 3 256 bytes
    return forced == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE : forced == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
         : forced == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
}

// A 3-d map over one operand: (contiguous dimension, strided dimension, batch entry).
bool encodeOperand(CUtensorMap* map, const void* base, int type, long long inner, long long outer, long long ld,
                   long long batch, long long batchStride, unsigned boxInner, unsigned boxOuter) {
    const int es = elemSizeOf(type);
    const CUtensorMapDataType dt = type == kF16    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                   : type == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                   : type == kF32  ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                   : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    const cuuint64_t dims[3] = {cuuint64_t(inner), cuuint64_t(outer), cuuint64_t(batch)};
    // a batch dimension of extent 1 still needs a legal stride
    const cuuint64_t strides[2] = {cuuint64_t(ld) * es, batch > 1 ? cuuint64_t(batchStride) * es : cuuint64_t(ld) * es * cuuint64_t(outer)};
    const cuuint32_t box[3] = {boxInner, boxOuter, 1};
    const cuuint32_t elemStrides[3] = {1, 1, 1};
    return encodeTiled()(map, dt, 3, const_cast<void*>(base), dims, strides, box, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, operandPromotion(), CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A 4-d map over an operand that is contiguous along m or n (`inner`), for extents that are whole chunks of 128 bytes:
// (element in chunk, k, chunk, batch entry). A box of `chunks` chunks by `boxOuter` rows of k lands in shared memory chunk after
// chunk, each as boxOuter rows of 128 bytes: the layout the per-chunk 3-d boxes produce, with one instruction instead of
// `chunks` (the producer's instruction count, not its bytes, is what a stage of MN-major operands costs more).
bool encodeChunked(CUtensorMap* map, const void* base, int type, long long inner, long long outer, long long ld, long long batch,
                   long long batchStride, unsigned chunkElems, unsigned boxOuter, unsigned chunks) {
    const int es = elemSizeOf(type);
    const CUtensorMapDataType dt = type == kF16    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                   : type == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                   : type == kF32  ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                   : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    const cuuint64_t dims[4] = {cuuint64_t(chunkElems), cuuint64_t(outer), cuuint64_t(inner / chunkElems), cuuint64_t(batch)};
    const cuuint64_t strides[3] = {cuuint64_t(ld) * es, cuuint64_t(chunkElems) * es,
                                   batch > 1 ? cuuint64_t(batchStride) * es : cuuint64_t(ld) * es * cuuint64_t(outer)};
    const cuuint32_t box[4] = {chunkElems, boxOuter, chunks, 1};
    const cuuint32_t elemStrides[4] = {1, 1, 1, 1};
    return encodeTiled()(map, dt, 4, const_cast<void*>(base), dims, strides, box, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int ummaKindOf(const Problem& p) {
    if (p.typeA != p.typeB) return -1;
    if ((p.typeA == kF16 || p.typeA == kBF16) && p.accType == kF32) return kKindF16;
    if (p.typeA == kS8 && p.accType == kS32) return kKindI8;
    // fp32 operands contiguous along m or n would need the 32-byte-atom swizzle (the only MN-major layout the
    // tensor cores take for 32-bit elements); they stay on the FFMA kernel
    if (p.typeA == kF32 && p.accType == kF32 && p.allowTf32 && p.transA && !p.transB) return kKindTf32;
    return -1;
}

// How many two-CTA clusters of this kernel the device runs at once (shared memory allows one CTA per SM, and the two
// CTAs of a cluster must sit in one GPC, so this can fall a little short of half the SM count).
template <int BN, bool PAIR, bool WIDE>
cudaError_t launchWith(const UmmaArgs& g, const CUtensorMap& mapA, const CUtensorMap& mapB, const CUtensorMap& mapD, const MirrorMaps& mirrors,
                       int slot, cudaStream_t stream) {
    using Plan = SmemPlan<BN, PAIR, WIDE>;
    DeviceInfo& d = deviceInfo();
    static std::mutex setupMutex;  // the first launch of a variant on a device sets it up; host threads may race to be first
    std::unique_lock<std::mutex> setup(setupMutex);
    if (!d.attrSet[slot]) {
        if (cudaError_t e = cudaFuncSetAttribute(ummaGemmKernel<BN, PAIR, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, Plan::kDynamicBytes);
            e != cudaSuccess)
            return e;
        if (PAIR) {
            cudaLaunchConfig_t probe{};
            probe.gridDim = dim3(unsigned(d.sms) / 2 * 2), probe.blockDim = dim3(kThreads), probe.dynamicSmemBytes = Plan::kDynamicBytes;
            cudaLaunchAttribute attr{};
            attr.id = cudaLaunchAttributeClusterDimension;
            attr.val.clusterDim.x = 2, attr.val.clusterDim.y = 1, attr.val.clusterDim.z = 1;
            probe.attrs = &attr, probe.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, ummaGemmKernel<BN, PAIR, WIDE>, &probe) != cudaSuccess || clusters < 1) {
                cudaGetLastError();
                clusters = d.sms / 2;
            }
            d.clusters[slot] = std::min(clusters, d.sms / 2);
        }
        d.attrSet[slot] = true;
    }
    setup.unlock();
    countLaunch();
    if (!PAIR) {
        const unsigned grid = unsigned(std::min<long long>(g.totalUnits, d.sms));
        ummaGemmKernel<BN, PAIR, WIDE><<<grid, kThreads, Plan::kDynamicBytes, stream>>>(g, mapA, mapB, mapD, mirrors);
        return cudaGetLastError();
    }
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(2u * unsigned(std::min<long long>(g.totalUnits, d.clusters[slot])));
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = Plan::kDynamicBytes;
    config.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2, attr.val.clusterDim.y = 1, attr.val.clusterDim.z = 1;
    config.attrs = &attr, config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, ummaGemmKernel<BN, PAIR, WIDE>, g, mapA, mapB, mapD, mirrors);
}

int pairClusters() {  // before the first launch has asked the device: half the SMs
    return deviceInfo().sms / 2;
}

}  // namespace

bool ummaEligible(const Problem& p) {
    if (p.k <= 0 || ummaKindOf(p) < 0) return false;
    if (!deviceInfo().sm100 || !encodeTiled()) return false;
    const int es = elemSizeOf(p.typeA);
    if (p.pointerArrays) {
        // The matrices' addresses are in device memory and are checked there (buildEntryMaps). What the host can see must
        // fit TMA, the entry maps need the handle's scratch memory, and the launch has to be worth its three kernels:
        // below about 2^24 flop the CUDA-core kernel is as fast.
        // (the caller then acquires that memory: 384 bytes per entry behind the counters; a batch too large for it stays
        // on the CUDA cores)
        return (p.lda * es) % 16 == 0 && (p.ldb * es) % 16 == 0 && size_t(p.batch) * 3 * sizeof(CUtensorMap) <= (size_t(32) << 20) &&
               2.0 * p.m * p.n * p.k * p.batch >= double(1 << 24) && p.m >= 32 && p.n >= 16;
    }
    const auto ok = [&](const void* ptr, long long ld, long long stride) {
        return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && (ld * es) % 16 == 0 &&
               (p.batch == 1 || stride == 0 || (stride * es) % 16 == 0);
    };
    return ok(p.A, p.lda, p.strideA) && ok(p.B, p.ldb, p.strideB);
}

bool ummaCanMirror(const Problem& p) {
    const EpilogueArgs& e = p.epi;
    const int esD = dtypeSize(e.typeD);
    const auto aligned = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
    if (e.pointerArrays || !aligned(e.D) || (e.ldd * esD) % 16 != 0 || ((long long)p.m * esD) % 16 != 0) return false;
    if (p.batch > 1 && (e.strideD == 0 || (e.strideD * esD) % 16 != 0)) return false;
    if (e.bias || e.activation != kActNone || e.roundBeforeBias || (e.typeC != e.typeD)) return false;  // the staged store forms only
    for (int q = 0; q < p.mirrorCount; ++q)
        if (!aligned(p.mirrorD[q])) return false;
    return true;
}

namespace {

// What a launch will look like: tile shape, pairing, epilogue variant and split count. Computed from the problem and the
// scratch memory on offer alone, so the dispatch layer can ask beforehand whether a call wants scratch memory at all.
struct UmmaPlan {
    int bn = 0;
    bool pair = false, wide = false;
    int splits = 1;
    int tilesM = 0, tilesN = 0;
    long long totalTiles = 0, kSlices = 0;
};

UmmaPlan planUmma(const Problem& p, size_t scratchBytes) {
    const int es = elemSizeOf(p.typeA);
    DeviceInfo& d = deviceInfo();
    UmmaPlan plan;
    // Tile shape: the candidate that needs the least time by a simple model. The main loop is bound by how fast operand
    // slices arrive from L2, so the cost of a candidate is its number of waves over the machine times the rows of 128
    // bytes one CTA fetches per k slice: 128 + BN for a CTA on its own, 128 + BN / 2 in a two-CTA pair (tile 256 x BN).
    const int mnBoxElems = kSliceBytes / es;  // an MN-major operand arrives in boxes of 128 bytes of m or n
    // forced choices exist only in a measurement build (measure.h)
    static const int forcedBn = measureKnob("VKZB_UMMA_BN", 0), forcedPair = measureKnob("VKZB_UMMA_PAIR", -1);
    static const int forcedSplits = measureKnob("VKZB_UMMA_SPLITS", 0);
    const long long kSlices = (p.k + kSliceBytes / es - 1) / (kSliceBytes / es);
    int bn = 0;
    bool pair = false;
    long long best = -1;
    for (int usePair = 1; usePair >= 0; --usePair) {
        if (forcedPair >= 0 && usePair != forcedPair) continue;
        for (int cand : {256, 128, 64}) {
            if (usePair && cand == 64) continue;
            if (forcedBn && cand != forcedBn) continue;
            const int ctaB = usePair ? cand / 2 : cand;
            if (p.transB && ctaB % mnBoxElems != 0) continue;  // int8 B^T: a box holds 128 columns
            const long long units = (long long)((p.m + (usePair ? 255 : 127)) / (usePair ? 256 : 128)) * ((p.n + cand - 1) / cand) * p.batch;
            const long long slots = usePair ? pairClusters() : d.sms;
            // plus a fixed cost per tile, in k slices: filling the pipeline and the accumulator hand-over (dearer between two CTAs)
            const long long slicesPerTile = kSlices + (usePair ? 6 : 3);
            const long long cost = (units + slots - 1) / slots * slicesPerTile * (kBM + ctaB);
            if (best < 0 || cost < best) best = cost, bn = cand, pair = usePair != 0;
        }
    }
    if (!bn) bn = p.transB && mnBoxElems > 64 ? 128 : 64, pair = false;  // forced values that fit nothing: smallest legal tile
    static const int forcedWide = measureKnob("VKZB_UMMA_WIDE", -1);
    // few k slices per tile: the launch is bound by writing D, so it takes the variant with more epilogue buffers
    // (measured at 4096 x 4096 x k, f16: k = 512, 8 slices, 29.1 us wide against 30.7; k = 1024, 16 slices, 38.8 against 35.4)
    const bool wide = forcedWide >= 0 ? forcedWide != 0 : kSlices <= 8;
    plan.bn = bn, plan.pair = pair, plan.wide = wide, plan.kSlices = kSlices;
    plan.tilesM = (p.m + (pair ? 255 : 127)) / (pair ? 256 : 128), plan.tilesN = (p.n + bn - 1) / bn;
    plan.totalTiles = (long long)plan.tilesM * plan.tilesN * p.batch;
    // Splitting along k through scratch memory. Measured, it pays for a small result with a long k, where the
    // tiles leave most SMs idle (4096 x 16 x 11008 f16: 50 -> 27 us; 512 x 512 x 16384 int8: 37 -> 19 us), and costs
    // time once the accumulators that travel through scratch memory are megabytes (4096 x 512 x 11008: 31 -> 43 us; that
    // main loop is bound by fetching its operands, which a split does not speed up). So: results of at most 2 MiB of
    // accumulators, all units in one wave, at least 8 k slices per split, as many splits (up to 4) as that allows.
    const long long halfTiles = plan.totalTiles * (pair ? 2 : 1), slots = pair ? pairClusters() : d.sms;
    const size_t room = scratchBytes > kSplitKCounters * sizeof(unsigned) ? scratchBytes - kSplitKCounters * sizeof(unsigned) : 0;
    const auto allowed = [&](int s) {
        return !wide && p.mirrorCount == 0 && !p.pointerArrays && kSlices / s >= 8 && halfTiles <= kSplitKCounters && size_t(halfTiles) * s * bn * kBM * 4 <= room;
    };
    if (forcedSplits > 1) {
        if (allowed(forcedSplits)) plan.splits = forcedSplits;
    } else if (!forcedSplits && (long long)p.m * p.n * p.batch * 4 <= (2 << 20)) {
        for (int s = 4; s > 1 && plan.splits == 1; --s)
            if (plan.totalTiles * s <= slots && allowed(s)) plan.splits = s;
    }
    return plan;
}

}  // namespace

bool ummaWantsScratch(const Problem& p, size_t scratchBytesOnOffer) { return planUmma(p, scratchBytesOnOffer).splits > 1; }

cudaError_t launchUmma(const Problem& p) {
    if (p.pointerArrays && (!p.scratch || p.scratchBytes < kSplitKCounters * sizeof(unsigned) + 256 + size_t(p.batch) * 3 * sizeof(CUtensorMap)))
        return cudaErrorInvalidValue;  // the dispatch layer hands pointer-array batches over only with scratch memory for their maps
    const int kind = ummaKindOf(p);
    const int es = elemSizeOf(p.typeA);
    const UmmaPlan plan = planUmma(p, p.scratch ? p.scratchBytes : 0);
    const int bn = plan.bn, splits = plan.splits;
    const bool pair = plan.pair, wide = plan.wide;
    UmmaArgs g{};
    g.m = p.m, g.n = p.n, g.k = p.k, g.batch = p.batch;
    g.tilesM = plan.tilesM, g.tilesN = plan.tilesN;
    // Raster. By default groups of 8 rows of pair tiles (16 of single ones): about as many tile rows as tile columns among the
    // tiles in flight. Products that are many groups tall AND many tiles wide (8192^3: 32 x 32 pair tiles) do better with the k
    // direction alternating between a CTA's units (producerLoop), which lets the A panels of a group survive in L2 from wave
    // to wave, and then with taller groups, so that every B panel is fetched once per group and there are half as many groups
    // (8192^3 f16: on one box 0.806 ms forward, 0.796 alternating; on another, alternating, 8 rows 0.857 ms, 12 rows 0.853,
    // 16 rows 0.846, 24 rows 0.86, 32 rows 0.88). Tall, narrow products with a long k lose by both (32768^3 in calls of
    // 2048 columns: 57.4 ms against 59.4 - 59.6), so they keep the default.
    const bool wideRaster = pair && plan.tilesM >= 32 && plan.tilesN >= 16;
    g.groupM = pair ? (wideRaster ? 16 : 8) : 16;
    g.serpentine = wideRaster;
    if (const int forcedGroup = measureKnob("VKZB_UMMA_GROUP_M", 0)) g.groupM = forcedGroup;
    if (const int forcedDirection = measureKnob("VKZB_UMMA_SERPENTINE", -1); forcedDirection >= 0) g.serpentine = forcedDirection;
    g.totalTiles = plan.totalTiles;
    g.splits = splits;
    g.totalUnits = g.totalTiles * splits;
    g.splitCounters = static_cast<unsigned*>(p.scratch);
    g.splitPartials = static_cast<unsigned*>(p.scratch) + kSplitKCounters;
    g.sliceElems = kSliceBytes / es;
    g.numKSlices = (p.k + g.sliceElems - 1) / g.sliceElems;
    g.kind = kind;
    g.mnMajorA = !p.transA;  // op(A) = A: stored m x k, m contiguous
    g.mnMajorB = p.transB;   // op(B) = B^T: stored n x k, n contiguous
    const unsigned format = kind == kKindF16 ? (p.typeA == kBF16 ? 1u : 0u) : kind == kKindTf32 ? 2u : 1u /* signed 8-bit */;
    const unsigned cFormat = kind == kKindI8 ? 2u : 1u;  // s32 : f32
    g.idesc = cFormat << 4 | format << 7 | format << 10 | unsigned(g.mnMajorA) << 15 | unsigned(g.mnMajorB) << 16 |
              unsigned(bn >> 3) << 17 | unsigned((pair ? 2 * kBM : kBM) >> 4) << 24;
    // stride offset 1024 bytes (8 rows of 128 bytes), descriptor version 1, 128-byte swizzle
    g.descHi = (1024u >> 4) | 1u << 14 | 2u << 29;
    const unsigned mnBoxBytes = unsigned(g.sliceElems) * kSliceBytes;  // slice-length rows of 128 bytes
    const unsigned mnKStep = (32u / es / 8u) * (1024u >> 4);          // k groups of 8 rows per MMA
    g.lboA = g.mnMajorA ? mnBoxBytes >> 4 : 1u;
    g.lboB = g.mnMajorB ? mnBoxBytes >> 4 : 1u;
    g.kStepA = g.mnMajorA ? mnKStep : 32u >> 4;
    g.kStepB = g.mnMajorB ? mnKStep : 32u >> 4;
    g.boxElemsA = g.boxElemsB = kSliceBytes / es;
    g.boxBytesA = g.boxBytesB = int(mnBoxBytes);
    g.boxesA = g.mnMajorA ? kBM / g.boxElemsA : 1;
    const int ctaB = pair ? bn / 2 : bn;  // B rows one CTA stages
    g.boxesB = g.mnMajorB ? ctaB / g.boxElemsB : 1;
    g.batchMulA = p.batch > 1 && p.strideA != 0 && !p.pointerArrays;
    g.batchMulB = p.batch > 1 && p.strideB != 0 && !p.pointerArrays;
    g.epi = p.epi;
    // Pointer arrays: the maps encoded here are templates (placeholder address: the scratch block, which is 256-byte aligned);
    // buildEntryMaps makes one set per batch entry from them, in scratch memory behind the counters and the flag word.
    unsigned* const entryFlag = p.pointerArrays ? static_cast<unsigned*>(p.scratch) + kSplitKCounters : nullptr;
    CUtensorMap* const entryMaps = p.pointerArrays ? reinterpret_cast<CUtensorMap*>(static_cast<char*>(p.scratch) + kSplitKCounters * sizeof(unsigned) + 256) : nullptr;
    const void* const baseA = p.pointerArrays ? p.scratch : p.A;
    const void* const baseB = p.pointerArrays ? p.scratch : p.B;
    void* const baseD = p.pointerArrays ? p.scratch : p.epi.D;
    g.entryMaps = entryMaps, g.entryFlag = entryFlag, g.entrySerial = p.launchSerial;

    CUtensorMap mapA, mapB;
    const long long batchA = g.batchMulA ? p.batch : 1, batchB = g.batchMulB ? p.batch : 1;
    static const bool noChunks = measureKnob("VKZB_UMMA_NO_CHUNKS", 0) != 0;
    g.chunkedA = g.mnMajorA && !noChunks && g.boxesA > 1 && p.m % g.boxElemsA == 0;
    g.chunkedB = g.mnMajorB && !noChunks && g.boxesB > 1 && p.n % g.boxElemsB == 0;
    // (a driver that refuses the 4-d view leaves the operand on its per-chunk boxes)
    if (g.chunkedA && !encodeChunked(&mapA, baseA, p.typeA, p.m, p.k, p.lda, batchA, p.strideA, g.boxElemsA, g.sliceElems, g.boxesA)) g.chunkedA = 0;
    if (g.chunkedB && !encodeChunked(&mapB, baseB, p.typeB, p.n, p.k, p.ldb, batchB, p.strideB, g.boxElemsB, g.sliceElems, g.boxesB)) g.chunkedB = 0;
    const bool okA = g.chunkedA || (g.mnMajorA ? encodeOperand(&mapA, baseA, p.typeA, p.m, p.k, p.lda, batchA, p.strideA, g.boxElemsA, g.sliceElems)
                                               : encodeOperand(&mapA, baseA, p.typeA, p.k, p.m, p.lda, batchA, p.strideA, g.sliceElems, kBM));
    const bool okB = g.chunkedB || (g.mnMajorB ? encodeOperand(&mapB, baseB, p.typeB, p.n, p.k, p.ldb, batchB, p.strideB, g.boxElemsB, g.sliceElems)
                                               : encodeOperand(&mapB, baseB, p.typeB, p.k, p.n, p.ldb, batchB, p.strideB, g.sliceElems, ctaB));
    if (!okA || !okB) return cudaErrorInvalidValue;

    // D through TMA when every address the bulk stores start at is 16-byte aligned; otherwise direct stores.
    // (With beta != 0 and C another matrix than D, C's type must be D's: the staged form reads C as D's type.)
    CUtensorMap mapD{};
    const EpilogueArgs& e = p.epi;
    const int esD = dtypeSize(e.typeD);
    // TMA clips a store at the tensor's edge in units of 16 bytes, so a column length that is not a multiple of 16 bytes
    // would let it write into the padding between m and ldd: those shapes keep the direct stores too.
    g.tmaStore = (e.ldd * esD) % 16 == 0 && ((long long)p.m * esD) % 16 == 0 &&
                 (e.pointerArrays || ((reinterpret_cast<uintptr_t>(e.D) & 15) == 0 && (p.batch == 1 || (e.strideD * esD) % 16 == 0) && (p.batch == 1 || e.strideD != 0)));
    if (measureKnob("VKZB_UMMA_DIRECT_STORE", 0)) g.tmaStore = 0;
    MirrorMaps mirrors{};
    g.mirrorCount = 0;
    if (g.tmaStore) {
        const CUtensorMapDataType dt = e.typeD == kF16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : e.typeD == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                       : e.typeD == kS32 ? CU_TENSOR_MAP_DATA_TYPE_INT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
        const cuuint64_t dims[3] = {cuuint64_t(p.m), cuuint64_t(p.n), cuuint64_t(e.pointerArrays ? 1 : p.batch)};
        const cuuint64_t strides[2] = {cuuint64_t(e.ldd) * esD, p.batch > 1 && !e.pointerArrays ? cuuint64_t(e.strideD) * esD : cuuint64_t(e.ldd) * esD * cuuint64_t(p.n)};
        const cuuint32_t box[3] = {cuuint32_t(kBM), cuuint32_t(kStepCols), 1}, ones[3] = {1, 1, 1};
        const auto encode = [&](CUtensorMap* map, void* base) {
            return encodeTiled()(map, dt, 3, base, dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                 CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
        };
        if (!encode(&mapD, baseD)) g.tmaStore = 0;
        for (int q = 0; g.tmaStore && q < p.mirrorCount; ++q) {
            if (!encode(&mirrors.map[q], p.mirrorD[q])) return cudaErrorInvalidValue;
            g.mirrorCount = q + 1;
        }
    }
    if (p.mirrorCount > 0 && g.mirrorCount != p.mirrorCount) return cudaErrorInvalidValue;  // never skip mirrors silently

    if (p.pointerArrays) {
        if (!g.tmaStore) mapD = mapA;  // never used; the builder copies three maps whatever they hold
        buildEntryMaps<<<(p.batch + 127) / 128, 128, 0, p.stream>>>(mapA, mapB, mapD, static_cast<const void* const*>(p.A), static_cast<const void* const*>(p.B),
                                                                     static_cast<void* const*>(e.D), p.batch, g.tmaStore, entryMaps, entryFlag, p.launchSerial);
        countLaunch();
        if (cudaError_t err = cudaGetLastError(); err != cudaSuccess) return err;
    }

    static const bool logChoice = [] { const char* v = std::getenv("VKZB_LOG"); return v && !std::strcmp(v, "debug"); }();
    if (logChoice)
        std::fprintf(stderr, "vkzb: umma tile %d x %d%s, %lld tiles, %d k slices in %d splits, %s store, chunked loads A %d B %d\n", pair ? 256 : 128, bn, pair ? (wide ? " (two-CTA pairs, wide epilogue)" : " (two-CTA pairs)") : (wide ? " (wide epilogue)" : ""),
                     g.totalTiles, g.numKSlices, splits, g.tmaStore ? "TMA" : "direct", g.chunkedA, g.chunkedB);
    setLastPlan(bn | (pair ? 1 << 10 : 0) | (wide ? 1 << 11 : 0) | splits << 12);
    if (wide) {
        if (pair) return bn == 256 ? launchWith<256, true, true>(g, mapA, mapB, mapD, mirrors, 8, p.stream) : launchWith<128, true, true>(g, mapA, mapB, mapD, mirrors, 9, p.stream);
        if (bn == 256) return launchWith<256, false, true>(g, mapA, mapB, mapD, mirrors, 5, p.stream);
        if (bn == 128) return launchWith<128, false, true>(g, mapA, mapB, mapD, mirrors, 6, p.stream);
        return launchWith<64, false, true>(g, mapA, mapB, mapD, mirrors, 7, p.stream);
    }
    if (pair) return bn == 256 ? launchWith<256, true, false>(g, mapA, mapB, mapD, mirrors, 3, p.stream) : launchWith<128, true, false>(g, mapA, mapB, mapD, mirrors, 4, p.stream);
    if (bn == 256) return launchWith<256, false, false>(g, mapA, mapB, mapD, mirrors, 0, p.stream);
    if (bn == 128) return launchWith<128, false, false>(g, mapA, mapB, mapD, mirrors, 1, p.stream);
    return launchWith<64, false, false>(g, mapA, mapB, mapD, mirrors, 2, p.stream);
}

const unsigned* ummaEntryFlag(const Problem& p) { return p.pointerArrays && p.scratch ? static_cast<const unsigned*>(p.scratch) + kSplitKCounters : nullptr; }

int ummaDeviceStatus() {
    unsigned status = 0;
    if (cudaMemcpyFromSymbol(&status, g_ummaStatus, sizeof status) != cudaSuccess) return -1;
    return int(status);
}

}  // namespace vkzb
