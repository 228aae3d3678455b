// vkzbSgemmStaticScratch: the split-k fp32 product on scratch memory that is part of the library image.
//
// Some users of this library hand every byte of device memory to their own pool when they start (an inference server
// sized to the model it serves) or run in a phase where cudaMalloc is off limits because it synchronises the whole device
// (a latency-bound serving loop). A cuBLAS handle of this library allocates its split-k scratch memory at the first call
// that wants to split, which is exactly what such a caller cannot allow. For them the same kernel (sgemmKernel, SPLITK form,
// k_sgemm.cu) runs on a file-scope device array: present on every GPU that loads this module for as long as the process
// lives, never allocated or freed by a call. This file is linked into libcublas.so.12 only, so a process carries one copy
// of the array per GPU however many of this repository's libraries it loads.
#include <algorithm>
#include <cstdio>

#include "gemm_problem.h"

namespace {
// Room for the arrival counters and 4 MiB of partial tiles: products of up to 256 tiles of 64 x 64 (m * n up to about one
// million results, for instance 1024 x 1024), cut into as many k slices as still fit.
constexpr size_t kStaticPartialBytes = size_t(4) << 20;
constexpr size_t kStaticCounterBytes = vkzb::kSplitKCounters * sizeof(unsigned);
constexpr size_t kStaticScratchBytes = kStaticCounterBytes + kStaticPartialBytes;
static __device__ __align__(256) unsigned char g_staticSplitKScratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void* g_staticScratchAddress[kMaxDevices] = {};  // the array's address on each device, looked up once (racing threads store the same value)
}  // namespace

extern "C" __attribute__((visibility("default"))) int vkzbSgemmStaticScratch(cudaStream_t stream, int transa, int transb, int m, int n, int k,
                                                                             const float* alpha, const float* A, int lda, const float* B,
                                                                             int ldb, const float* beta, float* C, int ldc) {
    using namespace vkzb;
    enum { kSuccess = 0, kNotInitialized = 1, kInvalidValue = 7, kExecutionFailed = 13, kNotSupported = 15 };  // cublasStatus_t values
    if (m < 0 || n < 0 || k < 0 || !alpha || !beta || unsigned(transa) > 2u || unsigned(transb) > 2u) return kInvalidValue;
    const int rowsA = transa == 0 ? m : k, rowsB = transb == 0 ? k : n;
    if (lda < std::max(1, rowsA) || ldb < std::max(1, rowsB) || ldc < std::max(1, m)) return kInvalidValue;
    if (m == 0 || n == 0) return kSuccess;
    if (k == 0 || m == 1 || n == 1) return kNotSupported;  // this entry point is the tiled split-k product only
    const long long tiles = (long long)((m + 63) / 64) * ((n + 63) / 64);
    if (tiles > kSplitKCounters || sgemmSplitKScratchBytes(m, n, 1) > kStaticScratchBytes) {
        std::fprintf(stderr, "vkzbSgemmStaticScratch: a %d x %d result needs %zu bytes of scratch memory, the built-in array holds %zu "
                             "(products of up to 256 tiles of 64 x 64)\n", m, n, sgemmSplitKScratchBytes(m, n, 1), kStaticScratchBytes);
        return kInvalidValue;
    }
    // Set-up, once per device, with that device current: in host code the array's name is only a stand-in, so its device
    // address has to be asked for. The first call on a device does this; the lookup makes the driver load this module onto
    // the device, which is when the array's memory is reserved (and may synchronise the device): a caller with a quiet phase
    // to protect makes one call per device during start-up, before any stream capture.
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return kNotInitialized;
    if (!g_staticScratchAddress[device]) {
        void* address = nullptr;
        if (cudaGetSymbolAddress(&address, g_staticSplitKScratch) != cudaSuccess || !address) {
            cudaGetLastError();
            return kNotInitialized;
        }
        g_staticScratchAddress[device] = address;
    }
    void* scratch = g_staticScratchAddress[device];
    Problem p;
    p.transA = transa != 0, p.transB = transb != 0;
    p.m = m, p.n = n, p.k = k, p.batch = 1;
    p.A = A, p.B = B, p.typeA = p.typeB = kF32;
    p.lda = lda, p.ldb = ldb;
    p.accType = kF32;
    p.epi.D = C, p.epi.C = C;
    p.epi.ldd = p.epi.ldc = ldc;
    p.epi.typeD = p.epi.typeC = kF32;
    p.epi.scalars.type = kScalarF32;
    p.epi.scalars.alphaHost = double(*alpha), p.epi.scalars.betaHost = double(*beta);
    p.stream = stream;
    if (!sgemmEligible(p)) return kInvalidValue;  // A and B must be 4-byte aligned
    int splits = int(std::min<long long>(std::min<long long>(8, std::max<long long>(1, 2LL * sgemmSmCount() / tiles)), std::max(1, k / 64)));
    while (splits > 1 && sgemmSplitKScratchBytes(m, n, splits) > kStaticScratchBytes) --splits;
    // The array keeps what the last call left in it. The kernel returns every counter it used to zero, but a call that was
    // cut short (a failed launch further up the stream, a context torn down mid-kernel and rebuilt) would leave some set: the
    // counters this call is about to use are cleared in stream order first. The partial tiles need no clearing (every slot
    // that is read has been written by this call).
    if (cudaMemsetAsync(scratch, 0, size_t(tiles) * sizeof(unsigned), stream) != cudaSuccess) {
        cudaGetLastError();
        return kExecutionFailed;
    }
    return launchSgemmSplitK(p, splits, scratch) == cudaSuccess ? kSuccess : kExecutionFailed;
}
