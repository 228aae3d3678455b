// libcublas.so.12 entry points: handle state, argument validation and the choice of kernel family.
//
// Mirrors the behaviour of k0zi/Vulkanizer's dispatch layer (src/cublas/cublas.cpp:189-218 handle, :235-258
// scalars, :698-925 run, :931-1262 exports) behind the same C ABI, with the kernels underneath replaced by
// the hand-written sm_100a ones of this repository. Differences that are deliberate:
//   * alpha and beta in device pointer mode are read by the kernels, not copied to the host, so no call blocks
//     or breaks stream capture (the reference does a blocking copy per scalar, cublas.cpp:241-243);
//   * int8 operands with CUBLAS_COMPUTE_32I are served (int32 alpha/beta, exact int32 sums); the reference
//     answers NOT_SUPPORTED for them (cublas.cpp:178-185);
//   * there is one tensor-core kernel and no run-time race between kernels (cublas.cpp:644-696).
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <initializer_list>

#include <cuda_fp16.h>

#define VKZB_HAVE_CUDA_TYPES
#include <library_types.h>

#include "../../include/vkzb_cublas.h"
#include "../../include/vkzb_ext.h"
#include "blas_internal.h"

namespace vkzb {

static std::atomic<uint64_t> g_launches{0};
static thread_local int t_lastPath = VKZB_PATH_NONE;
static thread_local int t_lastPlan = 0;

void setLastPlan(int packed) { t_lastPlan = packed; }

void countLaunch(int n) { g_launches.fetch_add(uint64_t(n), std::memory_order_relaxed); }

static int envLevel() {
    static const int level = [] {
        const char* v = std::getenv("VKZB_LOG");
        return v && (!std::strcmp(v, "debug") || !std::strcmp(v, "trace")) ? 1 : 0;
    }();
    return level;
}

// VKZB_FORCE_PATH (a test aid, like the reference's VULKANIZER_GEMM_COOP switch; read once):
//   generic  every GEMM that is not a matrix-vector product goes to the CUDA-core tile kernel
//   no-umma  the tcgen05 kernel is skipped; fp32 still takes the FFMA kernel
static int forcedPath() {
    static const int forced = [] {
        const char* v = std::getenv("VKZB_FORCE_PATH");
        if (v && !std::strcmp(v, "generic")) return int(VKZB_PATH_GENERIC);
        if (v && !std::strcmp(v, "no-umma")) return -int(VKZB_PATH_UMMA);
        return 0;
    }();
    return forced;
}

int dtypeOf(cudaDataType t) {
    switch (t) {
    case CUDA_R_32F: return kF32;
    case CUDA_R_16F: return kF16;
    case CUDA_R_16BF: return kBF16;
    case CUDA_R_8I: return kS8;
    case CUDA_R_32I: return kS32;
    case CUDA_R_64F: return kF64;
    default: return kBadType;
    }
}

int scalarTypeOf(cublasComputeType_t compute) {
    switch (compute) {
    case CUBLAS_COMPUTE_16F:
    case CUBLAS_COMPUTE_16F_PEDANTIC: return kScalarF16;
    case CUBLAS_COMPUTE_64F:
    case CUBLAS_COMPUTE_64F_PEDANTIC: return kScalarF64;
    case CUBLAS_COMPUTE_32I:
    case CUBLAS_COMPUTE_32I_PEDANTIC: return kScalarS32;
    default: return kScalarF32;
    }
}

static double hostScalar(const void* p, int type) {
    switch (type) {
    case kScalarF16: {
        __half h;
        std::memcpy(&h, p, 2);
        return double(__half2float(h));
    }
    case kScalarS32: {
        int v;
        std::memcpy(&v, p, 4);
        return double(v);
    }
    case kScalarF64: {
        double v;
        std::memcpy(&v, p, 8);
        return v;
    }
    default: {
        float v;
        std::memcpy(&v, p, 4);
        return double(v);
    }
    }
}

bool fillScalars(ScalarArgs& s, const void* alpha, const void* beta, int type, bool devicePointers) {
    if (!alpha || !beta) return false;
    s.type = type;
    if (devicePointers) {
        s.alphaDev = alpha, s.betaDev = beta;
        s.alphaHost = s.betaHost = 0;
    } else {
        s.alphaDev = s.betaDev = nullptr;
        s.alphaHost = hostScalar(alpha, type);
        s.betaHost = hostScalar(beta, type);
    }
    return true;
}

static const char* pathName(int path) {
    static const char* const names[] = {"none", "scale", "generic", "gemv", "sgemm (ffma)", "umma (tcgen05)", "dgemm"};
    return path >= 0 && path <= VKZB_PATH_DGEMM ? names[path] : "?";
}

// The accumulator the operand types call for, or kBadType when the combination is not served.
static int accumulatorFor(int ta, int tb, int tc, cublasComputeType_t compute) {
    const auto isFloat = [](int t) { return t == kF32 || t == kF16 || t == kBF16; };
    if (isFloat(ta) && isFloat(tb) && isFloat(tc)) return scalarTypeOf(compute) == kScalarF32 || scalarTypeOf(compute) == kScalarF16 ? kF32 : kBadType;
    if (ta == kF64 && tb == kF64 && tc == kF64) return scalarTypeOf(compute) == kScalarF64 ? kF64 : kBadType;
    if (ta == kS8 && tb == kS8 && tc == kS32) return scalarTypeOf(compute) == kScalarS32 ? kS32 : kBadType;
    return kBadType;
}

// ---- host time per entry point (VKZB_PROFILE=1) ----
namespace {
constexpr int kApiSlots = 96;
struct ApiRow {
    std::atomic<const char*> name{nullptr};
    std::atomic<unsigned long long> calls{0}, ns{0};
};
ApiRow g_apiRows[kApiSlots];

void printApiTable() {
    int order[kApiSlots], used = 0;
    for (int i = 0; i < kApiSlots; ++i)
        if (g_apiRows[i].name.load() && g_apiRows[i].calls.load()) order[used++] = i;
    if (!used) return;
    std::sort(order, order + used, [](int a, int b) { return g_apiRows[a].ns.load() > g_apiRows[b].ns.load(); });
    std::fprintf(stderr, "vkzb: host time per entry point (VKZB_PROFILE)\n%12s %10s %10s  %s\n", "total ms", "calls", "mean us", "entry point");
    for (int i = 0; i < used; ++i) {
        const ApiRow& r = g_apiRows[order[i]];
        const double ns = double(r.ns.load()), calls = double(r.calls.load());
        std::fprintf(stderr, "%12.3f %10.0f %10.2f  %s\n", ns * 1e-6, calls, ns * 1e-3 / calls, r.name.load());
    }
}

bool profiling() {
    static const bool on = [] {
        const char* v = std::getenv("VKZB_PROFILE");
        const bool enabled = v && *v && std::strcmp(v, "0") != 0;
        if (enabled) std::atexit(printApiTable);
        return enabled;
    }();
    return on;
}

long long nowNs() { return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
}  // namespace

// `name` is a string literal (__func__): rows are found by pointer first, by text when another call site shares the name.
ApiScope::ApiScope(const char* name) : slot_(-1), start_(0) {
    if (!profiling()) return;
    for (int i = 0; i < kApiSlots; ++i) {
        const char* have = g_apiRows[i].name.load(std::memory_order_acquire);
        if (!have) {
            const char* expected = nullptr;
            if (g_apiRows[i].name.compare_exchange_strong(expected, name)) have = name;
            else have = expected;
        }
        if (have == name || !std::strcmp(have, name)) {
            slot_ = i;
            break;
        }
    }
    start_ = nowNs();
}

ApiScope::~ApiScope() {
    if (slot_ < 0) return;
    g_apiRows[slot_].calls.fetch_add(1, std::memory_order_relaxed);
    g_apiRows[slot_].ns.fetch_add((unsigned long long)(nowNs() - start_), std::memory_order_relaxed);
}

// ---- the handle's scratch memory ----
constexpr size_t kScratchBytes = kSplitKCounters * sizeof(unsigned) + (size_t(64) << 20);  // counters, then 64 MiB of partial tiles

// Makes the handle's scratch memory usable by a call on `stream`, allocating it at the first call that wants it. Returns
// false when the call has to do without: allocation failed, or a stream capture is under way and the memory is not there
// yet or would need ordering against another stream (neither an allocation nor a cross-stream wait belongs in a capture).
static bool acquireScratch(cublasHandle_t h, cudaStream_t stream) {
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &capture) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    const bool capturing = capture != cudaStreamCaptureStatusNone;
    if (!h->scratch) {
        if (h->scratchTried || capturing) return false;
        h->scratchTried = true;
        if (cudaMalloc(&h->scratch, kScratchBytes) != cudaSuccess || cudaMemset(h->scratch, 0, kSplitKCounters * sizeof(unsigned) + 256) != cudaSuccess ||  // the counters and the flag word behind them
            cudaEventCreateWithFlags(&h->scratchEvent, cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            if (h->scratch) cudaFree(h->scratch);
            h->scratch = nullptr;
            return false;
        }
        h->scratchBytes = kScratchBytes;
    }
    if (h->scratchUsed && h->scratchStream != stream) {
        // the last user ran on another stream: this call waits for it on the device, the host does not block
        if (capturing) return false;
        if (cudaEventRecord(h->scratchEvent, h->scratchStream) != cudaSuccess || cudaStreamWaitEvent(stream, h->scratchEvent, 0) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
    }
    h->scratchStream = stream, h->scratchUsed = true;
    return true;
}

void releaseScratch(cublasContext* h) {
    if (h->scratch) cudaFree(h->scratch);
    if (h->scratchEvent) cudaEventDestroy(h->scratchEvent);
    h->scratch = nullptr, h->scratchEvent = nullptr, h->scratchBytes = 0;
}

// Would this call split along k if it had the scratch memory? (Only then is the memory allocated or ordered.)
static bool wantsScratch(const Problem& p, bool umma) {
    if (umma) return ummaWantsScratch(p, kScratchBytes);
    return sgemmSplitKPlan(p, kScratchBytes) > 1;
}

// Picks the kernel family and launches. `p` is complete except for the stream.
cublasStatus_t dispatch(cublasHandle_t h, Problem& p, cudaStream_t stream) {
    p.stream = stream;
    p.scratch = nullptr, p.scratchBytes = 0;
    p.mirrorCount = 0;
    if (h->mirrorCount > 0 && !p.epi.pointerArrays) {
        const char* d = static_cast<const char*>(p.epi.D);
        if (d >= h->mirrorLocal && d < h->mirrorLocal + h->mirrorBytes) {
            p.mirrorCount = h->mirrorCount;
            for (int i = 0; i < h->mirrorCount; ++i) p.mirrorD[i] = h->mirrorBase[i] + (d - h->mirrorLocal);
            // only the tensor-core kernel with bulk stores can write mirrors; anything else must say so
            if (p.k == 0 || p.n == 1 || p.m == 1 || forcedPath() != 0 || !ummaEligible(p) || !ummaCanMirror(p)) return CUBLAS_STATUS_NOT_SUPPORTED;
        }
    }
    int path;
    cudaError_t err;
    if (p.k == 0) {
        path = VKZB_PATH_SCALE;
        err = launchScale(p);
    } else if (p.n == 1 || p.m == 1 || (forcedPath() == 0 && p.mirrorCount == 0 && gemvTakesFewColumns(p))) {
        path = VKZB_PATH_GEMV;
        err = launchGemv(p);
    } else if (forcedPath() == VKZB_PATH_GENERIC) {
        path = VKZB_PATH_GENERIC;
        err = launchGeneric(p);
    } else if (forcedPath() != -int(VKZB_PATH_UMMA) && p.pointerArrays && ummaEligible(p) && acquireScratch(h, stream)) {
        p.scratch = h->scratch, p.scratchBytes = h->scratchBytes;
        // Pointer arrays on the tensor cores: a kernel builds a tensor map per batch entry in the handle's scratch memory,
        // the tcgen05 kernel runs on them, and the CUDA-core kernel is queued behind it for the one case only the device can
        // see, matrices whose addresses TMA cannot take: exactly one of the two does the work.
        path = VKZB_PATH_UMMA;
        p.launchSerial = ++h->launchSerial ? h->launchSerial : ++h->launchSerial;  // never 0, the word's initial content
        err = launchUmma(p);
        if (err == cudaSuccess) err = launchGenericStandIn(p, ummaEntryFlag(p), p.launchSerial);
    } else if (forcedPath() != -int(VKZB_PATH_UMMA) && !p.pointerArrays && ummaEligible(p)) {
        path = VKZB_PATH_UMMA;
        if (wantsScratch(p, true) && acquireScratch(h, stream)) p.scratch = h->scratch, p.scratchBytes = h->scratchBytes;
        err = launchUmma(p);
    } else if (sgemmEligible(p)) {
        path = VKZB_PATH_SGEMM;
        if (wantsScratch(p, false) && acquireScratch(h, stream)) p.scratch = h->scratch, p.scratchBytes = h->scratchBytes;
        err = launchSgemm(p);
    } else {
        path = p.accType == kF64 ? VKZB_PATH_DGEMM : VKZB_PATH_GENERIC;
        err = launchGeneric(p);
    }
    t_lastPath = path;
    if (envLevel())
        std::fprintf(stderr, "vkzb: gemm %c%c m=%d n=%d k=%d types %d/%d/%d batch %d%s -> %s%s%s\n", p.transA ? 'T' : 'N',
                     p.transB ? 'T' : 'N', p.m, p.n, p.k, p.typeA, p.typeB, p.epi.typeD, p.batch,
                     p.pointerArrays ? " (arrays)" : "", pathName(path), err == cudaSuccess ? "" : ": ",
                     err == cudaSuccess ? "" : cudaGetErrorString(err));
    return err == cudaSuccess ? CUBLAS_STATUS_SUCCESS : CUBLAS_STATUS_EXECUTION_FAILED;
}

namespace {

struct Call {
    cublasOperation_t transa, transb;
    int m, n, k;
    const void* alpha;
    const void* A;
    cudaDataType ta;
    int lda;
    long long strideA;
    const void* B;
    cudaDataType tb;
    int ldb;
    long long strideB;
    const void* beta;
    void* C;
    cudaDataType tc;
    int ldc;
    long long strideC;
    int batch;
    bool pointerArrays;
    cublasComputeType_t compute;
};

// Validation order and results follow cublas.cpp:698-710.
cublasStatus_t run(cublasHandle_t h, const Call& c) {
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    if (c.m < 0 || c.n < 0 || c.k < 0 || c.batch < 0) return CUBLAS_STATUS_INVALID_VALUE;
    const int rowsA = c.transa == CUBLAS_OP_N ? c.m : c.k, rowsB = c.transb == CUBLAS_OP_N ? c.k : c.n;
    if (c.lda < std::max(1, rowsA) || c.ldb < std::max(1, rowsB) || c.ldc < std::max(1, c.m)) return CUBLAS_STATUS_INVALID_VALUE;
    if (unsigned(c.transa) > CUBLAS_OP_C || unsigned(c.transb) > CUBLAS_OP_C) return CUBLAS_STATUS_INVALID_VALUE;
    if (c.m == 0 || c.n == 0 || c.batch == 0) {
        t_lastPath = VKZB_PATH_NONE;
        return CUBLAS_STATUS_SUCCESS;
    }
    const int ta = dtypeOf(c.ta), tb = dtypeOf(c.tb), tc = dtypeOf(c.tc);
    const int acc = (ta == kBadType || tb == kBadType || tc == kBadType) ? kBadType : accumulatorFor(ta, tb, tc, c.compute);
    if (acc == kBadType) return CUBLAS_STATUS_NOT_SUPPORTED;

    Problem p;
    p.transA = c.transa != CUBLAS_OP_N, p.transB = c.transb != CUBLAS_OP_N;
    p.m = c.m, p.n = c.n, p.k = c.k, p.batch = c.batch;
    p.A = c.A, p.B = c.B, p.typeA = ta, p.typeB = tb;
    p.lda = c.lda, p.ldb = c.ldb, p.strideA = c.strideA, p.strideB = c.strideB;
    p.pointerArrays = c.pointerArrays;
    p.accType = acc;
    p.allowTf32 = h->math == CUBLAS_TF32_TENSOR_OP_MATH || c.compute == CUBLAS_COMPUTE_32F_FAST_TF32;
    p.epi.D = c.C, p.epi.C = c.C;
    p.epi.ldd = p.epi.ldc = c.ldc;
    p.epi.strideD = p.epi.strideC = c.strideC;
    p.epi.typeD = p.epi.typeC = tc;
    p.epi.pointerArrays = c.pointerArrays;
    if (!fillScalars(p.epi.scalars, c.alpha, c.beta, scalarTypeOf(c.compute), h->pointerMode == CUBLAS_POINTER_MODE_DEVICE))
        return CUBLAS_STATUS_INVALID_VALUE;
    return dispatch(h, p, h->stream);
}

bool fitsInt(std::initializer_list<int64_t> values) {
    for (int64_t v : values)
        if (v < INT32_MIN || v > INT32_MAX) return false;
    return true;
}

}  // namespace
}  // namespace vkzb

using namespace vkzb;

#pragma GCC visibility push(default)
extern "C" {

cublasStatus_t cublasCreate_v2(cublasHandle_t* handle) {
    VKZB_API_SCOPE();
    if (!handle) return CUBLAS_STATUS_INVALID_VALUE;
    // Binds to the context that is current (a driver-API one made by the caller, or the device's primary
    // one, which this call brings up if needed) as cublas.cpp:931-945 does.
    if (cudaFree(nullptr) != cudaSuccess) return CUBLAS_STATUS_NOT_INITIALIZED;
    auto* h = new (std::nothrow) cublasContext;
    if (!h) return CUBLAS_STATUS_ALLOC_FAILED;
    cudaGetDevice(&h->device);
    envLevel();
    forcedPath();
    *handle = h;  // no device memory yet: split-k scratch comes with the first call that wants it (acquireScratch)
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasDestroy_v2(cublasHandle_t handle) {
    VKZB_API_SCOPE();
    if (!handle) return CUBLAS_STATUS_NOT_INITIALIZED;
    releaseScratch(handle);
    delete handle;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasGetVersion_v2(cublasHandle_t, int* version) {
    if (!version) return CUBLAS_STATUS_INVALID_VALUE;
    *version = VKZB_CUBLAS_VERSION;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasGetProperty(libraryPropertyType type, int* value) {
    if (!value) return CUBLAS_STATUS_INVALID_VALUE;
    *value = type == MAJOR_VERSION ? VKZB_CUBLAS_VER_MAJOR : type == MINOR_VERSION ? VKZB_CUBLAS_VER_MINOR : VKZB_CUBLAS_VER_PATCH;
    return CUBLAS_STATUS_SUCCESS;
}

size_t cublasGetCudartVersion(void) { return CUDART_VERSION; }

cublasStatus_t cublasSetStream_v2(cublasHandle_t h, cudaStream_t stream) {
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    h->stream = stream;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasGetStream_v2(cublasHandle_t h, cudaStream_t* stream) {
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    if (!stream) return CUBLAS_STATUS_INVALID_VALUE;
    *stream = h->stream;
    return CUBLAS_STATUS_SUCCESS;
}

// The kernels need no workspace (TMEM holds the accumulators); the pointer is remembered and unused.
cublasStatus_t cublasSetWorkspace_v2(cublasHandle_t h, void* workspace, size_t bytes) {
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    h->workspace = workspace, h->workspaceBytes = bytes;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasSetPointerMode_v2(cublasHandle_t h, cublasPointerMode_t mode) {
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    if (mode != CUBLAS_POINTER_MODE_HOST && mode != CUBLAS_POINTER_MODE_DEVICE) return CUBLAS_STATUS_INVALID_VALUE;
    h->pointerMode = mode;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasGetPointerMode_v2(cublasHandle_t h, cublasPointerMode_t* mode) {
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    if (!mode) return CUBLAS_STATUS_INVALID_VALUE;
    *mode = cublasPointerMode_t(h->pointerMode);
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasSetSmCountTarget(cublasHandle_t h, int) { return h ? CUBLAS_STATUS_SUCCESS : CUBLAS_STATUS_NOT_INITIALIZED; }

// Accumulation is fp32 whatever the mode; CUBLAS_TF32_TENSOR_OP_MATH alone moves fp32 GEMMs from the FFMA
// kernel to TF32 tensor cores.
cublasStatus_t cublasSetMathMode(cublasHandle_t h, cublasMath_t mode) {
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    h->math = mode & ~CUBLAS_MATH_DISALLOW_REDUCED_PRECISION_REDUCTION;
    h->mathFlags = mode & CUBLAS_MATH_DISALLOW_REDUCED_PRECISION_REDUCTION;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasGetMathMode(cublasHandle_t h, cublasMath_t* mode) {
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    if (!mode) return CUBLAS_STATUS_INVALID_VALUE;
    *mode = cublasMath_t(h->math | h->mathFlags);
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasSetAtomicsMode(cublasHandle_t h, cublasAtomicsMode_t mode) {
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    h->atomics = mode;
    return CUBLAS_STATUS_SUCCESS;
}

cublasStatus_t cublasGetAtomicsMode(cublasHandle_t h, cublasAtomicsMode_t* mode) {
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    if (!mode) return CUBLAS_STATUS_INVALID_VALUE;
    *mode = cublasAtomicsMode_t(h->atomics);
    return CUBLAS_STATUS_SUCCESS;
}

const char* cublasGetStatusName(cublasStatus_t status) {
    switch (status) {
    case CUBLAS_STATUS_SUCCESS: return "CUBLAS_STATUS_SUCCESS";
    case CUBLAS_STATUS_NOT_INITIALIZED: return "CUBLAS_STATUS_NOT_INITIALIZED";
    case CUBLAS_STATUS_ALLOC_FAILED: return "CUBLAS_STATUS_ALLOC_FAILED";
    case CUBLAS_STATUS_INVALID_VALUE: return "CUBLAS_STATUS_INVALID_VALUE";
    case CUBLAS_STATUS_ARCH_MISMATCH: return "CUBLAS_STATUS_ARCH_MISMATCH";
    case CUBLAS_STATUS_MAPPING_ERROR: return "CUBLAS_STATUS_MAPPING_ERROR";
    case CUBLAS_STATUS_EXECUTION_FAILED: return "CUBLAS_STATUS_EXECUTION_FAILED";
    case CUBLAS_STATUS_INTERNAL_ERROR: return "CUBLAS_STATUS_INTERNAL_ERROR";
    case CUBLAS_STATUS_NOT_SUPPORTED: return "CUBLAS_STATUS_NOT_SUPPORTED";
    case CUBLAS_STATUS_LICENSE_ERROR: return "CUBLAS_STATUS_LICENSE_ERROR";
    }
    return "CUBLAS_STATUS_UNKNOWN";
}

const char* cublasGetStatusString(cublasStatus_t status) {
    switch (status) {
    case CUBLAS_STATUS_SUCCESS: return "success";
    case CUBLAS_STATUS_NOT_INITIALIZED: return "the library was not initialized";
    case CUBLAS_STATUS_ALLOC_FAILED: return "the resource allocation failed";
    case CUBLAS_STATUS_INVALID_VALUE: return "an invalid numeric value was used as an argument";
    case CUBLAS_STATUS_ARCH_MISMATCH: return "an absent device architectural feature is required";
    case CUBLAS_STATUS_MAPPING_ERROR: return "an access to GPU memory space failed";
    case CUBLAS_STATUS_EXECUTION_FAILED: return "the GPU program failed to execute";
    case CUBLAS_STATUS_INTERNAL_ERROR: return "an internal operation failed";
    case CUBLAS_STATUS_NOT_SUPPORTED: return "the functionality requested is not supported";
    case CUBLAS_STATUS_LICENSE_ERROR: return "license error";
    }
    return "unknown error";
}

cublasStatus_t cublasLoggerConfigure(int, int, int, const char*) { return CUBLAS_STATUS_SUCCESS; }

cublasStatus_t cublasSgemm_v2(cublasHandle_t h, cublasOperation_t transa, cublasOperation_t transb, int m, int n, int k,
                              const float* alpha, const float* A, int lda, const float* B, int ldb, const float* beta,
                              float* C, int ldc) {
    VKZB_API_SCOPE();
    return run(h, {transa, transb, m, n, k, alpha, A, CUDA_R_32F, lda, 0, B, CUDA_R_32F, ldb, 0, beta, C, CUDA_R_32F, ldc, 0,
                   1, false, CUBLAS_COMPUTE_32F});
}

cublasStatus_t cublasSgemmBatched(cublasHandle_t h, cublasOperation_t transa, cublasOperation_t transb, int m, int n, int k,
                                  const float* alpha, const float* const A[], int lda, const float* const B[], int ldb,
                                  const float* beta, float* const C[], int ldc, int batchCount) {
    VKZB_API_SCOPE();
    return run(h, {transa, transb, m, n, k, alpha, A, CUDA_R_32F, lda, 0, B, CUDA_R_32F, ldb, 0, beta,
                   const_cast<void*>(static_cast<const void*>(C)), CUDA_R_32F, ldc, 0, batchCount, true, CUBLAS_COMPUTE_32F});
}

cublasStatus_t cublasSgemmStridedBatched(cublasHandle_t h, cublasOperation_t transa, cublasOperation_t transb, int m, int n,
                                         int k, const float* alpha, const float* A, int lda, long long strideA,
                                         const float* B, int ldb, long long strideB, const float* beta, float* C, int ldc,
                                         long long strideC, int batchCount) {
    VKZB_API_SCOPE();
    return run(h, {transa, transb, m, n, k, alpha, A, CUDA_R_32F, lda, strideA, B, CUDA_R_32F, ldb, strideB, beta, C,
                   CUDA_R_32F, ldc, strideC, batchCount, false, CUBLAS_COMPUTE_32F});
}

cublasStatus_t cublasDgemm_v2(cublasHandle_t h, cublasOperation_t transa, cublasOperation_t transb, int m, int n, int k,
                              const double* alpha, const double* A, int lda, const double* B, int ldb, const double* beta,
                              double* C, int ldc) {
    VKZB_API_SCOPE();
    return run(h, {transa, transb, m, n, k, alpha, A, CUDA_R_64F, lda, 0, B, CUDA_R_64F, ldb, 0, beta, C, CUDA_R_64F, ldc, 0,
                   1, false, CUBLAS_COMPUTE_64F});
}

cublasStatus_t cublasDgemmBatched(cublasHandle_t h, cublasOperation_t transa, cublasOperation_t transb, int m, int n, int k,
                                  const double* alpha, const double* const A[], int lda, const double* const B[], int ldb,
                                  const double* beta, double* const C[], int ldc, int batchCount) {
    VKZB_API_SCOPE();
    return run(h, {transa, transb, m, n, k, alpha, A, CUDA_R_64F, lda, 0, B, CUDA_R_64F, ldb, 0, beta,
                   const_cast<void*>(static_cast<const void*>(C)), CUDA_R_64F, ldc, 0, batchCount, true, CUBLAS_COMPUTE_64F});
}

cublasStatus_t cublasDgemmStridedBatched(cublasHandle_t h, cublasOperation_t transa, cublasOperation_t transb, int m, int n,
                                         int k, const double* alpha, const double* A, int lda, long long strideA,
                                         const double* B, int ldb, long long strideB, const double* beta, double* C, int ldc,
                                         long long strideC, int batchCount) {
    VKZB_API_SCOPE();
    return run(h, {transa, transb, m, n, k, alpha, A, CUDA_R_64F, lda, strideA, B, CUDA_R_64F, ldb, strideB, beta, C,
                   CUDA_R_64F, ldc, strideC, batchCount, false, CUBLAS_COMPUTE_64F});
}

cublasStatus_t cublasGemmEx(cublasHandle_t h, cublasOperation_t transa, cublasOperation_t transb, int m, int n, int k,
                            const void* alpha, const void* A, cudaDataType Atype, int lda, const void* B, cudaDataType Btype,
                            int ldb, const void* beta, void* C, cudaDataType Ctype, int ldc, cublasComputeType_t computeType,
                            cublasGemmAlgo_t) {
    VKZB_API_SCOPE();
    return run(h, {transa, transb, m, n, k, alpha, A, Atype, lda, 0, B, Btype, ldb, 0, beta, C, Ctype, ldc, 0, 1, false,
                   computeType});
}

// Half-precision GEMM with half scalars (cublas.cpp:1123-1129).
cublasStatus_t cublasHgemm(cublasHandle_t h, cublasOperation_t transa, cublasOperation_t transb, int m, int n, int k,
                           const void* alpha, const void* A, int lda, const void* B, int ldb, const void* beta, void* C,
                           int ldc) {
    VKZB_API_SCOPE();
    return run(h, {transa, transb, m, n, k, alpha, A, CUDA_R_16F, lda, 0, B, CUDA_R_16F, ldb, 0, beta, C, CUDA_R_16F, ldc, 0,
                   1, false, CUBLAS_COMPUTE_16F});
}

cublasStatus_t cublasGemmBatchedEx(cublasHandle_t h, cublasOperation_t transa, cublasOperation_t transb, int m, int n, int k,
                                   const void* alpha, const void* const Aarray[], cudaDataType Atype, int lda,
                                   const void* const Barray[], cudaDataType Btype, int ldb, const void* beta,
                                   void* const Carray[], cudaDataType Ctype, int ldc, int batchCount,
                                   cublasComputeType_t computeType, cublasGemmAlgo_t) {
    VKZB_API_SCOPE();
    return run(h, {transa, transb, m, n, k, alpha, Aarray, Atype, lda, 0, Barray, Btype, ldb, 0, beta,
                   const_cast<void*>(static_cast<const void*>(Carray)), Ctype, ldc, 0, batchCount, true, computeType});
}

cublasStatus_t cublasGemmStridedBatchedEx(cublasHandle_t h, cublasOperation_t transa, cublasOperation_t transb, int m, int n,
                                          int k, const void* alpha, const void* A, cudaDataType Atype, int lda,
                                          long long strideA, const void* B, cudaDataType Btype, int ldb, long long strideB,
                                          const void* beta, void* C, cudaDataType Ctype, int ldc, long long strideC,
                                          int batchCount, cublasComputeType_t computeType, cublasGemmAlgo_t) {
    VKZB_API_SCOPE();
    return run(h, {transa, transb, m, n, k, alpha, A, Atype, lda, strideA, B, Btype, ldb, strideB, beta, C, Ctype, ldc,
                   strideC, batchCount, false, computeType});
}

cublasStatus_t cublasSgemmEx(cublasHandle_t h, cublasOperation_t transa, cublasOperation_t transb, int m, int n, int k,
                             const float* alpha, const void* A, cudaDataType Atype, int lda, const void* B,
                             cudaDataType Btype, int ldb, const float* beta, void* C, cudaDataType Ctype, int ldc) {
    VKZB_API_SCOPE();
    return run(h, {transa, transb, m, n, k, alpha, A, Atype, lda, 0, B, Btype, ldb, 0, beta, C, Ctype, ldc, 0, 1, false,
                   CUBLAS_COMPUTE_32F});
}

// Groups of pointer-array batches, each with its own shape, scalars and leading dimensions given in host
// arrays; the pointer arrays list every problem group after group (cublas.cpp:1221-1251).
cublasStatus_t cublasGemmGroupedBatchedEx(cublasHandle_t h, const cublasOperation_t transa_array[],
                                          const cublasOperation_t transb_array[], const int m_array[], const int n_array[],
                                          const int k_array[], const void* alpha_array, const void* const Aarray[],
                                          cudaDataType Atype, const int lda_array[], const void* const Barray[],
                                          cudaDataType Btype, const int ldb_array[], const void* beta_array,
                                          void* const Carray[], cudaDataType Ctype, const int ldc_array[], int group_count,
                                          const int group_size[], cublasComputeType_t computeType) {
    VKZB_API_SCOPE();
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    if (group_count < 0) return CUBLAS_STATUS_INVALID_VALUE;
    if (group_count && (!transa_array || !transb_array || !m_array || !n_array || !k_array || !alpha_array || !lda_array ||
                        !ldb_array || !beta_array || !ldc_array || !group_size))
        return CUBLAS_STATUS_INVALID_VALUE;
    const int st = scalarTypeOf(computeType);
    const size_t scalarBytes = st == kScalarF16 ? 2 : st == kScalarF64 ? 8 : 4;
    size_t first = 0;
    for (int g = 0; g < group_count; ++g) {
        if (group_size[g] < 0) return CUBLAS_STATUS_INVALID_VALUE;
        const void* alpha = static_cast<const char*>(alpha_array) + g * scalarBytes;
        const void* beta = static_cast<const char*>(beta_array) + g * scalarBytes;
        const cublasStatus_t s =
            run(h, {transa_array[g], transb_array[g], m_array[g], n_array[g], k_array[g], alpha, Aarray + first, Atype,
                    lda_array[g], 0, Barray + first, Btype, ldb_array[g], 0, beta,
                    const_cast<void*>(static_cast<const void*>(Carray + first)), Ctype, ldc_array[g], 0, group_size[g], true,
                    computeType});
        if (s != CUBLAS_STATUS_SUCCESS) return s;
        first += size_t(group_size[g]);
    }
    return CUBLAS_STATUS_SUCCESS;
}

// y = alpha op(A) x + beta y as the m = 1 GEMM y^T = x^T op(A)^T: the vector increments become leading
// dimensions and the matrix-vector kernel does the work (cublas.cpp:1143-1159).
cublasStatus_t cublasSgemv_v2(cublasHandle_t h, cublasOperation_t trans, int m, int n, const float* alpha, const float* A,
                              int lda, const float* x, int incx, const float* beta, float* y, int incy) {
    VKZB_API_SCOPE();
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    if (m < 0 || n < 0 || lda < std::max(1, m) || incx == 0 || incy == 0) return CUBLAS_STATUS_INVALID_VALUE;
    if (incx < 0 || incy < 0) return CUBLAS_STATUS_NOT_SUPPORTED;
    const bool t = trans != CUBLAS_OP_N;
    const int rows = t ? n : m, cols = t ? m : n;
    if (rows == 0) return CUBLAS_STATUS_SUCCESS;
    return run(h, {CUBLAS_OP_N, t ? CUBLAS_OP_N : CUBLAS_OP_T, 1, rows, cols, alpha, x, CUDA_R_32F, incx, 0, A, CUDA_R_32F, lda,
                   0, beta, y, CUDA_R_32F, incy, 0, 1, false, CUBLAS_COMPUTE_32F});
}

// The 64-bit forms accept what fits the 32-bit ones and refuse the rest (cublas.cpp:1161-1209).
cublasStatus_t cublasSgemm_v2_64(cublasHandle_t h, cublasOperation_t transa, cublasOperation_t transb, int64_t m, int64_t n,
                                 int64_t k, const float* alpha, const float* A, int64_t lda, const float* B, int64_t ldb,
                                 const float* beta, float* C, int64_t ldc) {
    if (!fitsInt({m, n, k, lda, ldb, ldc})) return CUBLAS_STATUS_NOT_SUPPORTED;
    return cublasSgemm_v2(h, transa, transb, int(m), int(n), int(k), alpha, A, int(lda), B, int(ldb), beta, C, int(ldc));
}

cublasStatus_t cublasSgemmStridedBatched_64(cublasHandle_t h, cublasOperation_t transa, cublasOperation_t transb, int64_t m,
                                            int64_t n, int64_t k, const float* alpha, const float* A, int64_t lda,
                                            long long strideA, const float* B, int64_t ldb, long long strideB,
                                            const float* beta, float* C, int64_t ldc, long long strideC, int64_t batchCount) {
    if (!fitsInt({m, n, k, lda, ldb, ldc, batchCount})) return CUBLAS_STATUS_NOT_SUPPORTED;
    return cublasSgemmStridedBatched(h, transa, transb, int(m), int(n), int(k), alpha, A, int(lda), strideA, B, int(ldb),
                                     strideB, beta, C, int(ldc), strideC, int(batchCount));
}

cublasStatus_t cublasDgemm_v2_64(cublasHandle_t h, cublasOperation_t transa, cublasOperation_t transb, int64_t m, int64_t n,
                                 int64_t k, const double* alpha, const double* A, int64_t lda, const double* B, int64_t ldb,
                                 const double* beta, double* C, int64_t ldc) {
    if (!fitsInt({m, n, k, lda, ldb, ldc})) return CUBLAS_STATUS_NOT_SUPPORTED;
    return cublasDgemm_v2(h, transa, transb, int(m), int(n), int(k), alpha, A, int(lda), B, int(ldb), beta, C, int(ldc));
}

cublasStatus_t cublasDgemmStridedBatched_64(cublasHandle_t h, cublasOperation_t transa, cublasOperation_t transb, int64_t m,
                                            int64_t n, int64_t k, const double* alpha, const double* A, int64_t lda,
                                            long long strideA, const double* B, int64_t ldb, long long strideB,
                                            const double* beta, double* C, int64_t ldc, long long strideC, int64_t batchCount) {
    if (!fitsInt({m, n, k, lda, ldb, ldc, batchCount})) return CUBLAS_STATUS_NOT_SUPPORTED;
    return cublasDgemmStridedBatched(h, transa, transb, int(m), int(n), int(k), alpha, A, int(lda), strideA, B, int(ldb),
                                     strideB, beta, C, int(ldc), strideC, int(batchCount));
}

cublasStatus_t cublasSgemv_v2_64(cublasHandle_t h, cublasOperation_t trans, int64_t m, int64_t n, const float* alpha,
                                 const float* A, int64_t lda, const float* x, int64_t incx, const float* beta, float* y,
                                 int64_t incy) {
    if (!fitsInt({m, n, lda, incx, incy})) return CUBLAS_STATUS_NOT_SUPPORTED;
    return cublasSgemv_v2(h, trans, int(m), int(n), alpha, A, int(lda), x, int(incx), beta, y, int(incy));
}

// ---- extensions (include/vkzb_ext.h) ----
uint64_t vkzbLaunchCount(void) { return g_launches.load(std::memory_order_relaxed); }
int vkzbLastPath(void) { return t_lastPath; }
int vkzbLastPlan(void) { return t_lastPlan; }
int vkzbDeviceStatus(void) {
    const int umma = ummaDeviceStatus();
    return umma ? umma : gemvDeviceStatus();
}

int vkzbSetOutputMirrors(void* handle, const void* localBase, size_t bytes, int count, void* const* mirrorBases) {
    auto* h = static_cast<cublasContext*>(handle);
    if (!h) return CUBLAS_STATUS_NOT_INITIALIZED;
    if (count < 0 || count > kMaxMirrors || (count > 0 && (!localBase || !mirrorBases || !bytes))) return CUBLAS_STATUS_INVALID_VALUE;
    for (int i = 0; i < count; ++i)
        if (!mirrorBases[i]) return CUBLAS_STATUS_INVALID_VALUE;
    h->mirrorCount = count;
    h->mirrorLocal = static_cast<const char*>(localBase);
    h->mirrorBytes = bytes;
    for (int i = 0; i < count; ++i) h->mirrorBase[i] = static_cast<char*>(mirrorBases[i]);
    return CUBLAS_STATUS_SUCCESS;
}

}  // extern "C"
#pragma GCC visibility pop
