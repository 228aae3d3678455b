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
    // Scratch memory owned by the handle (allocated at creation, like cuBLAS's own workspace): partial sums of split-k
    // products. One handle, one stream at a time: two calls that overlap on the GPU through the same handle would share it.
    void* scratch = nullptr;
    size_t scratchBytes = 0;
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
cublasStatus_t dispatch(cublasContext* h, Problem& p);

}  // namespace vkzb
