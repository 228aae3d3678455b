// Internal description of one GEMM call, shared by the dispatch layer and every kernel family.
//
// The public entry points (cublasSgemm_v2, cublasGemmEx, cublasGemmStridedBatchedEx, cublasLtMatmul, ...)
// fold their arguments into a Problem the way k0zi/Vulkanizer folds them into `struct Gemm`
// (src/cublas/cublas.cpp:260-281); the kernels read it through EpilogueArgs / ScalarArgs below.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace vkzb {

// Storage types a matrix can have. The numeric codes index small tables in the kernels.
enum DType : int { kF32 = 0, kF16 = 1, kBF16 = 2, kS8 = 3, kS32 = 4, kF64 = 5, kBadType = -1 };

// Type of alpha and beta: fixed by the compute type (cublas.cpp:235-258 reads 2, 4 or 8 bytes).
enum ScalarType : int { kScalarF32 = 0, kScalarF16 = 1, kScalarS32 = 2, kScalarF64 = 3 };

// kActDRelu / kActDGelu are the backward forms: the value is multiplied by the activation's derivative at the forward
// pass's input, which the caller hands in as the auxiliary matrix (a bit mask for ReLU, the input itself for GELU).
enum Activation : int { kActNone = 0, kActRelu = 1, kActGelu = 2, kActDRelu = 3, kActDGelu = 4 };

// What the auxiliary matrix of a cuBLASLt epilogue is (NVIDIA's CUBLASLT_EPILOGUE_*_AUX and D* forms; the reference refuses
// them, src/cublas/cublasLt.cpp:68-78).
//   kAuxWriteMask   ReLU forward: bit (row + col * auxLd) of the matrix is 1 where the value before ReLU was > 0
//   kAuxWriteInput  GELU forward: the value before GELU, in the auxiliary type
//   kAuxReadMask    ReLU backward: the bit mask a forward pass wrote
//   kAuxReadInput   GELU backward: the forward pass's input
enum AuxMode : int { kAuxNone = 0, kAuxWriteMask = 1, kAuxWriteInput = 2, kAuxReadMask = 3, kAuxReadInput = 4 };

constexpr int kMaxMirrors = 7;  // other buffers a result can be written to as well (the other GPUs of an 8-GPU box)

__host__ __device__ inline int dtypeSize(int t) {
    return t == kF32 || t == kS32 ? 4 : t == kF64 ? 8 : t == kS8 ? 1 : 2;
}

// alpha and beta as the kernels see them. In host pointer mode the values were read on the host and
// travel by value; in device pointer mode the kernel dereferences the pointers itself, so no call
// ever blocks on a device-to-host copy (the reference does one per scalar, cublas.cpp:241-243).
struct ScalarArgs {
    double alphaHost, betaHost;  // exact for every scalar type (f16, f32, s32, f64)
    const void* alphaDev;        // non-null: device pointer mode
    const void* betaDev;
    int type;                    // ScalarType
};

// Where and how results are written: D = act(alpha * acc + beta * C + bias).
struct EpilogueArgs {
    void* D;              // matrix, or device array of matrix pointers when pointerArrays
    const void* C;        // read only when beta != 0; equals D for the cuBLAS entry points
    long long ldd, ldc;
    long long strideD, strideC;  // elements, per batch entry
    int typeD, typeC;     // DType
    const void* bias;     // per-row vector of length m, or null
    long long biasStride; // elements, per batch entry
    int typeBias;
    int biasAlongN;       // 1: the bias vector has length n and is indexed by the column (row-order problems, run transposed)
    int activation;       // Activation
    void* aux;            // auxiliary matrix of the epilogue (see AuxMode), or null
    long long auxLd;      // leading dimension of the auxiliary matrix: in elements, or in bits for the ReLU mask (a multiple of 32)
    long long auxStride;  // per batch entry, same unit
    int typeAux;          // DType of a GELU input matrix
    int auxMode;          // AuxMode
    int roundBeforeBias;  // 1: round alpha*acc+beta*C to D's type before bias/activation, as a second pass over D would
    int pointerArrays;    // D (and C) are arrays of pointers indexed by the batch entry
    ScalarArgs scalars;
};

struct Problem {
    bool transA = false, transB = false;
    int m = 0, n = 0, k = 0, batch = 1;
    const void* A = nullptr;
    const void* B = nullptr;
    int typeA = kF32, typeB = kF32;
    long long lda = 0, ldb = 0;
    long long strideA = 0, strideB = 0;
    bool pointerArrays = false;  // A, B, D are device arrays of pointers
    int accType = kF32;          // kF32, kS32 or kF64: the accumulator
    bool allowTf32 = false;      // handle asked for CUBLAS_TF32_TENSOR_OP_MATH or compute type FAST_TF32
    EpilogueArgs epi{};
    int mirrorCount = 0;              // D is also written to these addresses (same layout), tile by tile
    void* mirrorD[kMaxMirrors] = {};
    void* scratch = nullptr;          // the handle's scratch memory (split-k partial sums); calls sharing it must not overlap
    size_t scratchBytes = 0;
    unsigned launchSerial = 0;          // pointer-array launches on the tensor cores: this launch's number on its handle (see ummaEntryFlag)
    cudaStream_t stream = nullptr;
};

// Kernel families (launchers return cudaError_t; the dispatch layer maps it to a cuBLAS status).
cudaError_t launchScale(const Problem& p);    // k = 0: D = act(beta * C + bias)
cudaError_t launchGeneric(const Problem& p);  // any types / leading dimensions / pointer arrays
// out[i] = sum_j M[i * strideI + j * strideJ] for i < count, j < length, per batch entry (bias gradients of cuBLASLt epilogues)
cudaError_t launchVectorSums(const void* M, int type, long long strideI, long long strideJ, long long batchStrideM, int count, int length,
                             void* out, int typeOut, long long batchStrideOut, int batch, cudaStream_t stream);
bool gemvTakesFewColumns(const Problem& p);   // n = 2: two right-hand sides for which the matrix-vector kernel streams A once
cudaError_t launchGemv(const Problem& p);     // m = 1 or n = 1 (or gemvTakesFewColumns)
bool sgemmEligible(const Problem& p);
cudaError_t launchSgemm(const Problem& p);    // fp32 FFMA (split along k through p.scratch when the product is small)
constexpr int kSplitKCounters = 4096;          // arrival counters at the start of split-k scratch memory
// Pointer-array launches on the tensor cores: the device word that holds p.launchSerial when the tensor-core kernel stood down
// (an entry's address does not suit TMA), and the CUDA-core stand-in that then does the work.
const unsigned* ummaEntryFlag(const Problem& p);
cudaError_t launchGenericStandIn(const Problem& p, const unsigned* runIfEquals, unsigned value);
size_t sgemmSplitKScratchBytes(int m, int n, int splits);
int sgemmSplitKPlan(const Problem& p, size_t scratchBytes);
cudaError_t launchSgemmSplitK(const Problem& p, int splits, void* scratch);
int sgemmSmCount();                           // SMs of the device that was current at the first call
bool ummaEligible(const Problem& p);
bool ummaCanMirror(const Problem& p);          // D and the mirrors can be written with bulk stores
bool ummaWantsScratch(const Problem& p, size_t scratchBytesOnOffer);  // the launch would split along k given that much scratch memory
cudaError_t launchUmma(const Problem& p);     // tcgen05 tensor cores
int ummaDeviceStatus();
int gemvDeviceStatus();                      // 0, or 16 after a bulk copy of the matrix-vector kernel never arrived

// Triangular solves and batched factorizations (k_solve.cu), T = float or double. Matrices are a pointer-array batch
// (`arrays`), or single matrices with batch = 1.
template <typename T>
cudaError_t launchTrsm(bool right, bool upper, bool trans, bool unit, int m, int n, double alpha, const void* A, long long lda, const void* B,
                       long long ldb, int batch, bool arrays, cudaStream_t stream);
template <typename T>
cudaError_t launchGetrf(int n, const void* A, long long lda, int* pivots, int* info, int batch, cudaStream_t stream);
template <typename T>
cudaError_t launchGetrs(bool trans, int n, int nrhs, const void* A, long long lda, const int* pivots, const void* B, long long ldb, int batch,
                        cudaStream_t stream);
template <typename T>
cudaError_t launchGeqrf(int m, int n, const void* A, long long lda, const void* tau, int batch, cudaStream_t stream);

void countLaunch(int n = 1);
void setLastPlan(int packed);  // what vkzbLastPlan() reports for this thread's most recent tensor-core launch

}  // namespace vkzb
