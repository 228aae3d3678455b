/*
 * Fused attention, exported by this repository's libcublas.so.12: O = softmax(scale Q K^T + mask) V without the score matrix
 * ever reaching memory.
 *
 * k0zi/Vulkanizer has no entry point of this kind: it meets attention below the runtime, where its driver layer recognises
 * PyTorch's memory-efficient attention kernels by name and runs a shader of its own for them (src/driver/attention.h;
 * tests/attention.cpp states the semantics those kernels have, which are the ones kept here: the mask conventions, rows
 * without a visible key giving 0, the natural-log logsumexp, grouped-query heads). A library that is entered through the
 * cuBLAS ABI sees only the two batched products of an unfused attention, so the fused form is offered as an extension that a
 * framework calls instead of those two products.
 */
#ifndef VKZB_ATTENTION_H
#define VKZB_ATTENTION_H

#ifndef VKZB_HAVE_CUDA_TYPES
typedef struct CUstream_st* cudaStream_t;
#endif

#ifdef __cplusplus
extern "C" {
#endif

/*
 * Element (b, h, i, d) of Q is q[b * qBatch + h * qHead + i * qRow + d], likewise for K, V and O: the head dimension is
 * contiguous, every other stride is given in elements and must be a multiple of 8 (16 bytes), as must the four base
 * addresses. [batch, sequence, head, dim] tensors (PyTorch's layout for these kernels) have row = heads * dim, head = dim;
 * one matrix per batch entry as in a strided-batched GEMM has heads = 1.
 */
typedef struct vkzbAttentionProblem {
    int dataType;          /* cudaDataType of Q, K, V and O: CUDA_R_16F (2) or CUDA_R_16BF (14); accumulation and softmax in fp32 */
    int batches, heads;
    int kvHeads;           /* K and V have this many heads; query head h reads head h / (heads / kvHeads) */
    int numQ, numK;        /* queries and keys per head */
    int headDim;           /* 64 or 128, the same for Q, K, V and O */
    int mask;              /* 0 none; 1 key j visible to query i when j <= i; 2 when j <= i + numK - numQ */
    float scale;           /* multiplies Q K^T before the softmax */
    const void* q; long long qRow, qHead, qBatch;
    const void* k; long long kRow, kHead, kBatch;
    const void* v; long long vRow, vHead, vBatch;
    void* o;       long long oRow, oHead, oBatch;
    float* logSumExp;      /* optional, [batches][heads][numQ]: log(sum_j exp(score_ij)); 0 for a row with no visible key */
} vkzbAttentionProblem;

/*
 * Asynchronous on `stream`. Returns a cublasStatus_t value: 0 on success, CUBLAS_STATUS_NOT_SUPPORTED (15) for a type, head
 * dimension or alignment outside the above, CUBLAS_STATUS_INVALID_VALUE (7) for a null pointer or a negative extent.
 * A row without a visible key (possible with mask 2 when numK < numQ) gives zeros.
 */
int vkzbAttentionForward(cudaStream_t stream, const vkzbAttentionProblem* problem);

/*
 * Device-side status word of the attention kernel on the current device: 0 while every bounded wait completed, else the
 * code of the wait that gave up (33 the loader, 34 the tensor-core issuer, 35 the softmax warps). Blocking; -1 on a CUDA error.
 */
int vkzbAttentionStatus(void);

#ifdef __cplusplus
}
#endif
#endif
