// Matrix-vector kernels for GEMMs with n = 1 or m = 1 (the decode shape): y = alpha M v + beta y.
//
// Same contract as k0zi/Vulkanizer's route and shader (src/cublas/cublas.cpp:736-780, src/cublas/shaders/gemv.comp:87-146):
// M is `rows` x `len` with arbitrary row and column strides, v has stride incv, y stride incy, each of
// f32 / f16 / bf16 (int8 with int32 sums), batches by stride or by pointer arrays.
//
// The work is one pass over M, so the kernel is bound by HBM bandwidth, and at decode sizes (tens of megabytes, ten
// microseconds) by how quickly a launch gets its whole share of the matrix in flight. When rows are contiguous along the
// reduction (op(A) = A^T for n = 1), 16-byte aligned and 16-bit, gemvRowsBulk runs one block of 16 warps per SM; each warp
// owns an 8 KB shared-memory stage that bulk asynchronous copies fill (one instruction moves a whole piece of a row and
// signals an mbarrier), so a warp has 8 KB on the way instead of the 2 KB its registers could hold, and the vector sits in
// shared memory. Measured, a launch costs  t = t0 + bytes / 6.1..6.5 TB/s  with t0 = 3.0 us, the time a chain of dependent
// 8 x 8 products takes per launch (2.0 us with programmatic stream serialisation, which this kernel asks for): the stream
// rate is the copy bandwidth of the part, and at 4096 x 4096 (33 MB) t0 is a quarter of the time.
// gemvRowsVec16 (a warp per row, 128-bit loads into registers, no shared memory) serves batches and rows the bulk copy
// cannot take. Any other layout takes the scalar or the strided kernel (a thread per row, coalesced when the rows are
// interleaved in memory).
#include <cstdio>
#include <cstdlib>

#include "epilogue.cuh"
#include "measure.h"

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
    int vectors;              // 1, or kMaxVectors right-hand sides sharing one pass over M (n = 2 of a GEMM)
    long long vectorStride;   // elements between them (ldb); result (r, j) goes to C(r, j)
    int overlap;  // bulk kernel: launched with programmatic stream serialisation (1), and asks L2 for its first rows before the wait (2)
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

// The same with the mixed-precision FMA of sm_100 (two 16-bit factors, fp32 addend and result, one rounding): the products
// and sums are bit for bit those of dot8, without the conversion instructions, which otherwise outnumber the FMAs two to one.
template <bool BF16>
__device__ __forceinline__ float dot8Mixed(const uint4& a, const uint4& b, float acc) {
    const unsigned aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if constexpr (BF16)
            asm("{\n\t.reg .b16 al, ah, bl, bh;\n\tmov.b32 {al, ah}, %1;\n\tmov.b32 {bl, bh}, %2;\n\t"
                "fma.rn.f32.bf16 %0, al, bl, %0;\n\tfma.rn.f32.bf16 %0, ah, bh, %0;\n\t}"
                : "+f"(acc)
                : "r"(aw[i]), "r"(bw[i]));
        else
            asm("{\n\t.reg .b16 al, ah, bl, bh;\n\tmov.b32 {al, ah}, %1;\n\tmov.b32 {bl, bh}, %2;\n\t"
                "fma.rn.f32.f16 %0, al, bl, %0;\n\tfma.rn.f32.f16 %0, ah, bh, %0;\n\t}"
                : "+f"(acc)
                : "r"(aw[i]), "r"(bw[i]));
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

// A launch with programmatic stream serialisation lets blocks of this kernel become resident while the kernel before it in
// the stream drains; they wait here until that kernel has completed and its writes are visible. Without the launch
// attribute both instructions do nothing.
__device__ __forceinline__ void waitForPriorKernel() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void releaseNextKernel() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Only a hint may come before that wait: it moves no data into the kernel, so it is right whatever the kernel before still
// writes, and the loads after the wait find the bytes in L2.
__device__ __forceinline__ void prefetchToL2(const void* p, unsigned bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
constexpr int kUnroll = 4;  // 16-byte loads in flight per lane (measured: 4 beats 1, 2, 8 and 16 from 4096 to 32000 rows)

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
    float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
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

// ---- bulk-copy kernel --------------------------------------------------------------------------------------------

constexpr int kBulkWarps = 16;  // of the kernel with the vector in registers
constexpr int kBulkMaxWarps = 24;  // of the kernel with the vector in shared memory
constexpr int kMaxVectors = 2;  // measured (4096 x n x 4096 f16): n = 2 10.8 us here against 15.5 on the tensor cores, n = 3 12.9,
                                // n = 4 14.7, and slower than the tensor cores from n = 3 on when the rows are 11008 long
constexpr int kPieceBytes = 8192;                   // one ring stage: a row of 4096 halves, or a piece of a longer one
constexpr int kSharedLimit = 227 * 1024;
constexpr unsigned long long kBulkWaitLimitNs = 2000000000ull;

__device__ unsigned g_gemvStatus;  // 0, or 1 once a wait for a bulk copy ran out of time (the launch's result is then incomplete)

__device__ __forceinline__ unsigned sharedAddr(const void* p) { return unsigned(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void bulkLoad(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

// True once the phase with `parity` has completed; false after two seconds, with the status word set.
__device__ __forceinline__ bool bulkWait(unsigned bar, unsigned parity) {
    unsigned long long start = 0;
    for (unsigned spins = 0;; ++spins) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
        if ((spins & 255u) == 255u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (start == 0) start = now;
            else if (now - start > kBulkWaitLimitNs) {
                atomicExch(&g_gemvStatus, 1u);
                return false;
            }
        }
    }
}

// One block per SM, rows dealt to blocks in equal contiguous shares and to a block's warps in turn. A warp owns `stages`
// ring stages and their mbarriers: lane 0 issues the copies, all lanes wait, multiply the piece with the matching piece of
// the vector (shared memory, loaded once per block) and, after __syncwarp, lane 0 refills the stage. No block-level barrier
// after start-up. Needs len % 8 == 0 and everything the 128-bit register kernel needs.
//
// The launch allows programmatic stream serialisation: when the kernel before this one in the stream lets its successor
// start early (this kernel does), a block becomes resident as soon as an SM has room, sets up its barriers, asks L2 for its
// first rows and only then waits for the kernel before it to complete; every load of data comes after that wait.
struct BulkShape {
    int warps, stages, pieceBytes, pieces, vectorBytes, prefetchRows, vectors;
    size_t sharedBytes() const { return size_t(vectorBytes) * vectors + size_t(warps) * stages * (pieceBytes + 8) + 8; }
};

template <bool BF16, int NV>
__global__ void __launch_bounds__(kBulkMaxWarps * 32) gemvRowsBulk(const GemvArgs g, const BulkShape shape) {
    extern __shared__ __align__(128) unsigned char shared[];
    const int stages = shape.stages, warps = shape.warps, pieceBytes = shape.pieceBytes, pieces = shape.pieces;
    unsigned char* vecShared = shared;
    unsigned char* ring = shared + shape.vectorBytes * NV;  // a multiple of 128
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const unsigned barBase = sharedAddr(ring + size_t(warps) * stages * pieceBytes);
    const unsigned vecBar = barBase + 8u * warps * stages;
    const int rowBytes = g.len * 2;
    const int firstRow = int((long long)g.rows * blockIdx.x / gridDim.x);
    const int endRow = int((long long)g.rows * (blockIdx.x + 1) / gridDim.x);
    const char* M = static_cast<const char*>(g.M);
    if (threadIdx.x == 0) {
        for (int i = 0; i <= warps * stages; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(barBase + 8u * i) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (g.overlap) {
        if (lane == 0)
            for (int row = firstRow + warp, n = 0; row < endRow && n < shape.prefetchRows; row += warps, ++n)
                prefetchToL2(M + (long long)row * g.rowStride * 2, unsigned(rowBytes));
        waitForPriorKernel();
        releaseNextKernel();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // the vector goes in pieces as well: one copy moves at most what the mbarrier's byte counter can take
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(vecBar), "r"(unsigned(rowBytes) * NV) : "memory");
        for (int j = 0; j < NV; ++j)
            for (int at = 0; at < rowBytes; at += 8192)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 sharedAddr(vecShared + j * shape.vectorBytes + at)),
                             "l"(static_cast<const char*>(g.v) + j * g.vectorStride * 2 + at), "r"(unsigned(min(8192, rowBytes - at))), "r"(vecBar)
                             : "memory");
    }
    const int myRows = (endRow - firstRow - warp + warps - 1) / warps;  // rows firstRow + warp, + warps, ...
    if (myRows <= 0) return;
    const int items = myRows * pieces;
    unsigned char* myRing = ring + size_t(warp) * stages * pieceBytes;
    const unsigned myBars = barBase + 8u * warp * stages;

    const auto issue = [&](int item) {  // lane 0 only
        const int r = item / pieces, piece = item - r * pieces;
        const int row = firstRow + warp + r * warps;
        const int stage = item % stages;
        bulkLoad(sharedAddr(myRing + stage * pieceBytes), M + ((long long)row * g.rowStride * 2 + (long long)piece * pieceBytes),
                 unsigned(min(pieceBytes, rowBytes - piece * pieceBytes)), myBars + 8u * stage);
    };
    if (lane == 0)
        for (int i = 0; i < min(stages, items); ++i) issue(i);
    if (!bulkWait(vecBar, 0)) return;

    Epilogue<float> epi;
    epi.init(g.epi, 0);
    float acc[NV][4] = {};
    int piece = 0, r = 0;
    for (int item = 0; item < items; ++item) {
        const int stage = item % stages;
        if (!bulkWait(myBars + 8u * stage, unsigned(item / stages) & 1u)) return;
        const uint4* a = reinterpret_cast<const uint4*>(myRing + stage * pieceBytes);
        const uint4* x = reinterpret_cast<const uint4*>(vecShared + piece * pieceBytes);
        const int vectorChunks = shape.vectorBytes / 16;  // uint4 between two vectors in shared memory
        const int chunks = min(pieceBytes, rowBytes - piece * pieceBytes) / 16;
        const auto fourChunks = [&](int c0) {  // chunks c0, c0 + 32, c0 + 64, c0 + 96 of the piece against every vector
            uint4 av[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) av[u] = a[c0 + 32 * u];
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                uint4 xv[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) xv[u] = x[j * vectorChunks + c0 + 32 * u];
#pragma unroll
                for (int u = 0; u < 4; ++u) acc[j][u] = dot8Mixed<BF16>(av[u], xv[u], acc[j][u]);
            }
        };
        int c = lane;
        if (chunks == kPieceBytes / 16) {
#pragma unroll
            for (int q = 0; q < kPieceBytes / 16 / 128; ++q) fourChunks(lane + 128 * q);
            c = chunks;
        }
        for (; c + 96 < chunks; c += 128) fourChunks(c);
        for (; c < chunks; c += 32) {
            const uint4 av = a[c];
#pragma unroll
            for (int j = 0; j < NV; ++j) acc[j][0] = dot8Mixed<BF16>(av, x[j * vectorChunks + c], acc[j][0]);
        }
        __syncwarp();
        if (lane == 0 && item + stages < items) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the reads above come before the copy that overwrites them
            issue(item + stages);
        }
        if (++piece == pieces) {
            const int row = firstRow + warp + r * warps;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                float sum = (acc[j][0] + acc[j][1]) + (acc[j][2] + acc[j][3]);
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
                if (lane == 0) {
                    if (NV == 1) storeY(epi, g.yIsRow, row, sum);
                    else epi.store(row, j, sum);
                }
                acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
            }
            piece = 0;
            ++r;
        }
    }
}

// How the bulk kernel is laid out for rows of `len` 16-bit values; warps = 0 when it cannot take the shape.
// Measured on 4096 x 4096 to 32000 x 4096: 16 warps with one stage each beat 8 x 3, 12 x 2, 20 x 1 and 24 x 1.
BulkShape bulkShape(int len, int vectors) {
    BulkShape shape{};
    shape.vectors = vectors;
    if (len % 8 != 0) return shape;
    const int rowBytes = len * 2;
    shape.vectorBytes = (rowBytes + 127) / 128 * 128;
    shape.pieces = (rowBytes + kPieceBytes - 1) / kPieceBytes;
    shape.pieceBytes = ((rowBytes + shape.pieces - 1) / shape.pieces + 511) / 512 * 512;  // equal pieces, whole warp-wide trips
    shape.stages = 1;
    shape.prefetchRows = 2;
    static const int firstWarps = measureKnob("VKZB_GEMV_BULK_WARPS", 16);
    for (shape.warps = firstWarps; shape.warps >= 8; shape.warps -= 4)
        if (shape.sharedBytes() <= size_t(kSharedLimit)) return shape;
    shape.warps = 0;  // a vector too long to sit in shared memory beside the ring
    return shape;
}

// ---- rows of up to 8 KB with the vector in registers ---------------------------------------------------------------------
//
// The decode shape proper: one right-hand side, rows of CHUNKS x 512 bytes (K = 4096 halves for CHUNKS = 16). Each lane keeps
// its CHUNKS 16-byte pieces of the vector in registers for the whole launch, so shared memory carries nothing but the ring,
// which takes all 227 KB: 28 rows of 8 KB. A 4096 x 4096 matrix gives a block of an 148-SM part 27 or 28 rows, so every byte
// the block will read is requested in its first microsecond and the launch lasts one memory latency plus the stream time,
// where a ring of one stage per warp (16 x 8 KB) needed two round trips (14 warps x 2 slots for 8 KB rows).
// Issuing the first loads before the wait for the prior kernel (safe only under a caller's promise that nothing in flight
// writes the matrix) was measured and gained under 3 %, so every load comes after the wait.
template <bool BF16, int CHUNKS, bool MIXED>
__global__ void __launch_bounds__(kBulkWarps * 32) gemvRowsResidentVector(const GemvArgs g, const int slotsPerWarp) {
    extern __shared__ __align__(128) unsigned char shared[];
    constexpr int kRowBytes = CHUNKS * 512;
    const int warps = blockDim.x / 32, warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int slots = warps * slotsPerWarp;
    const unsigned barBase = sharedAddr(shared + size_t(slots) * kRowBytes);
    const int firstRow = int((long long)g.rows * blockIdx.x / gridDim.x);
    const int rows = int((long long)g.rows * (blockIdx.x + 1) / gridDim.x) - firstRow;
    const char* M = static_cast<const char*>(g.M) + (long long)firstRow * g.rowStride * 2;
    if (threadIdx.x == 0) {
        for (int i = 0; i < slots; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(barBase + 8u * i) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    // Warp w multiplies block-local rows w, w + warps, ...; its j-th row goes through its own slot j % slotsPerWarp, so a
    // slot is waited for, read and refilled by one warp, in that order.
    const int myRows = (rows - warp + warps - 1) / warps;
    unsigned char* myRing = shared + size_t(warp) * slotsPerWarp * kRowBytes;
    const unsigned myBars = barBase + 8u * warp * slotsPerWarp;
    const auto issue = [&](int j) {  // this warp's j-th row into its slot
        const int slot = j % slotsPerWarp;
        bulkLoad(sharedAddr(myRing + size_t(slot) * kRowBytes), M + (long long)(warp + j * warps) * g.rowStride * 2, unsigned(kRowBytes), myBars + 8u * slot);
    };
    const int first = min(slotsPerWarp, myRows);
    if (g.overlap) {
        if (lane < first) prefetchToL2(M + (long long)(warp + lane * warps) * g.rowStride * 2, unsigned(kRowBytes));
        waitForPriorKernel();
        releaseNextKernel();
    }
    if (lane < first) issue(lane);
    if (myRows <= 0) return;
    // the vector: this lane's pieces, straight from global memory (8 KB that every warp of the machine reads: L2 serves it)
    uint4 x[CHUNKS];
    const uint4* v = reinterpret_cast<const uint4*>(g.v);
#pragma unroll
    for (int q = 0; q < CHUNKS; ++q) x[q] = __ldg(v + lane + 32 * q);
    for (int j = 0; j < myRows; ++j) {
        const int slot = j % slotsPerWarp;
        if (!bulkWait(myBars + 8u * slot, unsigned(j / slotsPerWarp) & 1u)) return;
        const uint4* a = reinterpret_cast<const uint4*>(myRing + size_t(slot) * kRowBytes) + lane;
        float acc[4] = {};
#pragma unroll
        for (int q = 0; q < CHUNKS; q += 2) {  // two 16-byte loads in flight per lane: with the vector in 64 registers more would spill
            uint4 av[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) av[u] = a[32 * (q + u)];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if constexpr (MIXED) acc[(q + u) % 4] = dot8Mixed<BF16>(av[u], x[q + u], acc[(q + u) % 4]);
                else acc[(q + u) % 4] = dot8<BF16>(av[u], x[q + u], acc[(q + u) % 4]);
            }
        }
        __syncwarp();
        if (lane == 0 && j + slotsPerWarp < myRows) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the reads above come before the copy that overwrites them
            issue(j + slotsPerWarp);
        }
        float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
        if (lane == 0) {  // the epilogue's state is set up here, once per row, rather than held in registers across the loop
            Epilogue<float> epi;
            epi.init(g.epi, 0);
            storeY(epi, g.yIsRow, firstRow + warp + j * warps, sum);
        }
    }
}

// The kernel above serves rows of 2, 4 or 8 KB (K = 1024, 2048, 4096 16-bit values).
int residentVectorChunks(int len) { return len == 4096 ? 16 : len == 2048 ? 8 : len == 1024 ? 4 : 0; }

template <bool BF16, int CHUNKS, bool MIXED>
cudaError_t launchResidentVectorFor(const Problem& p, const GemvArgs& g) {
    static bool prepared[64] = {};
    int device = 0, sms = 0;
    if (cudaError_t e = cudaGetDevice(&device); e != cudaSuccess) return e;
    if (cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device); e != cudaSuccess) return e;
    if (device < 64 && !prepared[device]) {
        if (cudaError_t e = cudaFuncSetAttribute(gemvRowsResidentVector<BF16, CHUNKS, MIXED>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSharedLimit);
            e != cudaSuccess)
            return e;
        prepared[device] = true;
    }
    // Sixteen warps per SM with one slot each. Measured on 4096 x 4096 and 11008 x 4096 f16 (one block of 16 warps per SM):
    // 16 x 1 slots 6.6 / 15.1 us, 14 x 2 7.8 / 15.8, 12 x 2 7.7 / 15.6, 8 x 3 8.1 / 15.2: the multiply, not the bytes in
    // flight, is what a block waits for, so warps count for more than slots. The same 16 warps as four blocks of four
    // (blocks of the next launch then find room beside those of this one): 6.6 / 14.6 us; that form serves matrices with
    // at least 64 rows per SM, where it gains 3 %.
    const int rowBytes = CHUNKS * 512, maxSlots = (kSharedLimit - 1024) / (rowBytes + 8);
    static const int forcedBlocks = measureKnob("VKZB_GEMV_BLOCKS_PER_SM", 0);
    const int blocksPerSm = forcedBlocks ? forcedBlocks : g.rows >= 64 * sms ? 4 : 1;
    const int blocks = std::min(sms * blocksPerSm, g.rows);
    int warps = kBulkWarps / blocksPerSm, slotsPerWarp = 1;
    static const int forcedWarps = measureKnob("VKZB_GEMV_WARPS", 0), forcedSlots = measureKnob("VKZB_GEMV_SLOTS", 0);
    if (forcedWarps) warps = forcedWarps, slotsPerWarp = forcedSlots ? forcedSlots : std::max(1, maxSlots / blocksPerSm / warps);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(warps * 32);
    cfg.dynamicSmemBytes = size_t(warps) * slotsPerWarp * (rowBytes + 8);
    cfg.stream = p.stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = g.overlap ? 1 : 0;
    countLaunch();
    return cudaLaunchKernelEx(&cfg, gemvRowsResidentVector<BF16, CHUNKS, MIXED>, g, slotsPerWarp);
}

template <bool BF16>
cudaError_t launchResidentVector(const Problem& p, const GemvArgs& g, int chunks) {
    static const bool mixed = measureKnob("VKZB_GEMV_MIXED", 1) != 0;  // measurement builds can fall back to convert-then-FMA
    if (!mixed) return chunks == 16 ? launchResidentVectorFor<BF16, 16, false>(p, g) : cudaErrorInvalidValue;
    switch (chunks) {
    case 16: return launchResidentVectorFor<BF16, 16, true>(p, g);
    case 8: return launchResidentVectorFor<BF16, 8, true>(p, g);
    case 4: return launchResidentVectorFor<BF16, 4, true>(p, g);
    default: return cudaErrorInvalidValue;
    }
}

template <bool BF16, int NV>
cudaError_t launchBulkFor(const Problem& p, const GemvArgs& g, const BulkShape& shape) {
    static bool prepared[64] = {};
    int device = 0, sms = 0;
    if (cudaError_t e = cudaGetDevice(&device); e != cudaSuccess) return e;
    if (cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device); e != cudaSuccess) return e;
    if (device < 64 && !prepared[device]) {
        if (cudaError_t e = cudaFuncSetAttribute(gemvRowsBulk<BF16, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSharedLimit); e != cudaSuccess)
            return e;
        prepared[device] = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(std::min(sms, g.rows));
    cfg.blockDim = dim3(shape.warps * 32);
    cfg.dynamicSmemBytes = shape.sharedBytes();
    cfg.stream = p.stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = g.overlap ? 1 : 0;
    countLaunch();
    return cudaLaunchKernelEx(&cfg, gemvRowsBulk<BF16, NV>, g, shape);
}

template <bool BF16>
cudaError_t launchBulk(const Problem& p, const GemvArgs& g, const BulkShape& shape) {
    switch (shape.vectors) {
    case 1: return launchBulkFor<BF16, 1>(p, g, shape);
    case 2: return launchBulkFor<BF16, 2>(p, g, shape);
    default: return cudaErrorInvalidValue;
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

// A product with two columns whose matrix the bulk-copy kernel can stream: the columns of B are two right-hand sides of one
// pass over A. (Below about 16 columns a GEMM is bound by reading A, and the tensor-core kernel takes half as long again for
// that pass: 4096 x n x 4096 f16 took 15.5 us for n = 2 .. 64 against 9.5 us for n = 1. More than two right-hand sides make
// this kernel's conversions and FMAs the bound.)
// 0: plain launches; 2 (the default): programmatic serialisation, the blocks start before the prior kernel has ended
static int overlapMode() {
    static const int mode = measureKnob("VKZB_GEMV_OVERLAP", 2);
    return mode;
}

bool gemvTakesFewColumns(const Problem& p) {
    const auto aligned16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
    static const bool disabled = measureKnob("VKZB_GEMV_NO_FEW_COLUMNS", 0) != 0;  // measurement builds only
    if (disabled || p.n < 2 || p.n > kMaxVectors || p.m < 64 || p.batch != 1 || p.pointerArrays || p.accType != kF32) return false;
    if (!p.transA || p.transB || p.typeA != p.typeB || (p.typeA != kF16 && p.typeA != kBF16)) return false;
    if (p.k < 8 || p.k % 8 != 0 || p.lda % 8 != 0 || p.ldb % 8 != 0 || !aligned16(p.A) || !aligned16(p.B)) return false;
    return bulkShape(p.k, p.n).warps != 0;
}

cudaError_t launchGemv(const Problem& p) {
    GemvArgs g{};
    g.len = p.k;
    g.pointerArrays = p.pointerArrays;
    g.epi = p.epi;
    g.vectors = 1;
    if (p.n > 1 && p.m > 1) {  // gemvTakesFewColumns(p) holds
        g.M = p.A, g.v = p.B, g.typeM = p.typeA, g.typeV = p.typeB;
        g.rows = p.m, g.rowStride = p.lda, g.colStride = 1, g.incv = 1, g.yIsRow = 0;
        g.vectors = p.n, g.vectorStride = p.ldb;
        g.overlap = overlapMode();
        const BulkShape shape = bulkShape(g.len, g.vectors);
        if (!shape.warps) return cudaErrorInvalidValue;
        return g.typeM == kBF16 ? launchBulk<true>(p, g, shape) : launchBulk<false>(p, g, shape);
    }
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
    g.overlap = overlapMode();
    static const bool rowsOnly = measureKnob("VKZB_GEMV_ROWS_ONLY", 0) != 0;  // measurement builds: never the bulk-copy kernel
    const BulkShape shape = vec16 && p.batch == 1 && !rowsOnly ? bulkShape(g.len, 1) : BulkShape{};
    static const bool noResident = measureKnob("VKZB_GEMV_NO_RESIDENT", 0) != 0;  // measurement builds only
    if (shape.warps && !noResident && residentVectorChunks(g.len) && g.rows >= 64)
        return g.typeM == kBF16 ? launchResidentVector<true>(p, g, residentVectorChunks(g.len)) : launchResidentVector<false>(p, g, residentVectorChunks(g.len));
    if (shape.warps) return g.typeM == kBF16 ? launchBulk<true>(p, g, shape) : launchBulk<false>(p, g, shape);
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

int gemvDeviceStatus() {
    unsigned status = 0;
    if (cudaMemcpyFromSymbol(&status, g_gemvStatus, sizeof status) != cudaSuccess) return -1;
    return status ? 16 : 0;
}

}  // namespace vkzb
