// Shared between the cuBLAS and cuBLASLt entry points: the handle and the path from a folded Problem to a launch.
#pragma once

#include "gemm_problem.h"

// The library context behind cublasHandle_t and cublasLtHandle_t (one type, so either handle serves both
// libraries, as in k0zi/Vulkanizer: include/cublas/cublasLt.h:16-17, src/cublas/cublasLt.cpp:137-138).
// Plain fields: a handle is not to be shared between threads without the caller's own locking.
struct cublasContext {
    cudaStream_t stream = nullptr;
    int math = 0;         // cublasMath_t without the reduced-precision-reduction flag
    int mathFlags = 0;
    int pointerMode = 0;  // cublasPointerMode_t
    int atomics = 0;
    int device = 0;
    void* workspace = nullptr;
    size_t workspaceBytes = 0;
    // Scratch memory owned by the handle: arrival counters and partial sums of split-k products. Nothing is allocated until
    // the first call that wants to split (and never during a stream capture); a handle whose allocation failed simply does not
    // split. Calls that use it from a different stream than the last one that did are ordered behind that one with an event.
    void* scratch = nullptr;
    size_t scratchBytes = 0;
    bool scratchTried = false;
    cudaStream_t scratchStream = nullptr;  // stream of the last call that used the scratch memory
    bool scratchUsed = false;
    cudaEvent_t scratchEvent = nullptr;
    unsigned launchSerial = 0;  // numbers the pointer-array launches that use the scratch memory's flag word
    // output mirrors (vkzbSetOutputMirrors): results inside [mirrorLocal, mirrorLocal + mirrorBytes) are also written there
    const char* mirrorLocal = nullptr;
    size_t mirrorBytes = 0;
    int mirrorCount = 0;
    char* mirrorBase[vkzb::kMaxMirrors] = {};
};

namespace vkzb {

int dtypeOf(cudaDataType t);
int scalarTypeOf(cublasComputeType_t compute);
bool fillScalars(ScalarArgs& s, const void* alpha, const void* beta, int type, bool devicePointers);
// Picks the kernel family for `p` and launches it on `stream` (the handle's own for cuBLAS calls, the call's for cuBLASLt).
cublasStatus_t dispatch(cublasContext* h, Problem& p, cudaStream_t stream);
void releaseScratch(cublasContext* h);  // at handle destruction

// Host time per exported entry point, printed at exit when VKZB_PROFILE=1 (the counterpart of the reference's
// VULKANIZER_PROFILE=1 table, src/common/log.cpp:44-74). A scope object at the top of an entry point does the timing.
class ApiScope {
public:
    explicit ApiScope(const char* name);
    ~ApiScope();
private:
    int slot_;
    long long start_;
};
#define VKZB_API_SCOPE() ::vkzb::ApiScope vkzbApiScope_(__func__)

}  // namespace vkzb
