/*
 * C ABI of the libnccl.so.2 built by this repository: collectives between the ranks (processes or communicators) of ONE
 * machine, moved over NVLink / NVSwitch peer memory. Names, signatures and enum values are NCCL's documented ones (exported
 * unversioned, as NCCL's own library does), so a program built against NVIDIA's nccl.h binds unchanged. Each declaration
 * names the k0zi/Vulkanizer entry point it replaces as `src/nccl/nccl.cpp:<line>`.
 *
 * How it differs from the reference underneath the ABI: the reference synchronises the stream, copies the operand to the
 * host and exchanges it through POSIX shared memory (src/nccl/nccl.cpp:335-418). Here only buffer addresses travel through
 * shared memory (as CUDA IPC handles); data moves GPU to GPU with stream-ordered peer copies and device kernels, ranks
 * meeting on sequence-number flags in peer-mapped memory, so a collective is asynchronous on its stream. Every wait, on the
 * host and on the device, is bounded; a wait that gives up surfaces as ncclRemoteError / ncclSystemError.
 * When two ranks of a communicator share one GPU (the reference's tests do that) kernels of different ranks may not wait on
 * one another on that GPU, so the ranks meet on the host instead and the collective synchronises its stream, like the
 * reference's.
 *
 * Reductions accumulate floating point in double and integers in 64 bits, in rank order, so every rank receives identical
 * bits (the property src/nccl/nccl.cpp:9-10, 152-182 promises).
 */
#ifndef VKZB_NCCL_H
#define VKZB_NCCL_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef VKZB_HAVE_CUDA_TYPES
typedef struct CUstream_st* cudaStream_t;
#endif

#define NCCL_MAJOR 2
#define NCCL_MINOR 32
#define NCCL_PATCH 3
#define NCCL_VERSION_CODE (NCCL_MAJOR * 10000 + NCCL_MINOR * 100 + NCCL_PATCH)
#define NCCL_UNIQUE_ID_BYTES 128
#define NCCL_SPLIT_NOCOLOR (-1)

typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[NCCL_UNIQUE_ID_BYTES]; } ncclUniqueId;
typedef struct ncclConfig_v22800 ncclConfig_t; /* accepted and ignored */

typedef enum {
    ncclSuccess = 0, ncclUnhandledCudaError = 1, ncclSystemError = 2, ncclInternalError = 3, ncclInvalidArgument = 4,
    ncclInvalidUsage = 5, ncclRemoteError = 6, ncclInProgress = 7, ncclNumResults = 8
} ncclResult_t;
typedef enum { ncclSum = 0, ncclProd = 1, ncclMax = 2, ncclMin = 3, ncclAvg = 4, ncclNumOps = 5 } ncclRedOp_t;
typedef enum { ncclScalarDevice = 0, ncclScalarHostImmediate = 1 } ncclScalarResidence_t;
typedef enum {
    ncclInt8 = 0, ncclUint8 = 1, ncclInt32 = 2, ncclUint32 = 3, ncclInt64 = 4, ncclUint64 = 5, ncclFloat16 = 6, ncclFloat32 = 7,
    ncclFloat64 = 8, ncclBfloat16 = 9, ncclFloat8e4m3 = 10, ncclFloat8e5m2 = 11, ncclNumTypes = 12
} ncclDataType_t;

ncclResult_t ncclGetVersion(int* version);                                                          /* nccl.cpp:497 */
ncclResult_t ncclGetUniqueId(ncclUniqueId* uniqueId);                                               /* nccl.cpp:503 */
ncclResult_t ncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId commId, int rank);         /* nccl.cpp:511 */
ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId commId, int rank, ncclConfig_t* config); /* nccl.cpp:518 */
ncclResult_t ncclCommInitAll(ncclComm_t* comms, int ndev, const int* devlist);                      /* nccl.cpp:528 */
ncclResult_t ncclCommFinalize(ncclComm_t comm);                                                     /* nccl.cpp:545 */
ncclResult_t ncclCommDestroy(ncclComm_t comm);                                                      /* nccl.cpp:547 */
ncclResult_t ncclCommAbort(ncclComm_t comm);                                                        /* nccl.cpp:554 */
const char* ncclGetErrorString(ncclResult_t result);                                                /* nccl.cpp:593 */
const char* ncclGetLastError(ncclComm_t comm);                                                      /* nccl.cpp:607 */
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* asyncError);                      /* nccl.cpp:609 */
ncclResult_t ncclCommCount(const ncclComm_t comm, int* count);                                      /* nccl.cpp:615 */
ncclResult_t ncclCommCuDevice(const ncclComm_t comm, int* device);                                  /* nccl.cpp:621 */
ncclResult_t ncclCommUserRank(const ncclComm_t comm, int* rank);                                    /* nccl.cpp:627 */
ncclResult_t ncclCommRegister(const ncclComm_t comm, void* buff, size_t size, void** handle);       /* nccl.cpp:634 */
ncclResult_t ncclCommDeregister(const ncclComm_t comm, void* handle);                               /* nccl.cpp:639 */
ncclResult_t ncclMemAlloc(void** ptr, size_t size);                                                 /* nccl.cpp:641 */
ncclResult_t ncclMemFree(void* ptr);                                                                /* nccl.cpp:648 */

ncclResult_t ncclReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, int root,
                        ncclComm_t comm, cudaStream_t stream);                                      /* nccl.cpp:667 */
ncclResult_t ncclBroadcast(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, int root,
                           ncclComm_t comm, cudaStream_t stream);                                   /* nccl.cpp:672 */
ncclResult_t ncclBcast(void* buff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream); /* nccl.cpp:677 */
ncclResult_t ncclAllReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op,
                           ncclComm_t comm, cudaStream_t stream);                                   /* nccl.cpp:681 */
ncclResult_t ncclReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount, ncclDataType_t datatype, ncclRedOp_t op,
                               ncclComm_t comm, cudaStream_t stream);                               /* nccl.cpp:686 */
/* The gather that follows the N-sharded GEMM: rank r's `sendcount` elements land at recvbuff + r * sendcount on every rank. */
ncclResult_t ncclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount, ncclDataType_t datatype, ncclComm_t comm,
                           cudaStream_t stream);                                                    /* nccl.cpp:691 */
ncclResult_t ncclAlltoAll(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclComm_t comm,
                          cudaStream_t stream);                                                     /* nccl.cpp:696 */
ncclResult_t ncclGather(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm,
                        cudaStream_t stream);                                                       /* nccl.cpp:701 */
/* Point to point: the n-th send of a rank to a peer matches that peer's n-th receive from the rank. A send completes on its
 * stream when the receiver has copied the data. Issue a send and the receive it depends on in one group (as NCCL asks). */
ncclResult_t ncclSend(const void* sendbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm,
                      cudaStream_t stream);                                                         /* nccl.cpp:706 */
ncclResult_t ncclRecv(void* recvbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm,
                      cudaStream_t stream);                                                         /* nccl.cpp:711 */
/* A sum whose contributions are multiplied by a per-rank scalar first; usable wherever a ncclRedOp_t is until destroyed. */
ncclResult_t ncclRedOpCreatePreMulSum(ncclRedOp_t* op, void* scalar, ncclDataType_t datatype, ncclScalarResidence_t residence,
                                      ncclComm_t comm);                                             /* nccl.cpp:650 */
ncclResult_t ncclRedOpDestroy(ncclRedOp_t op, ncclComm_t comm);                                     /* nccl.cpp:662 */
/* Ranks passing the same color form a new communicator, ordered by (key, rank); NCCL_SPLIT_NOCOLOR yields none. */
ncclResult_t ncclCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* newcomm, ncclConfig_t* config); /* nccl.cpp:561 */
/* Operations issued between GroupStart and GroupEnd are started together at GroupEnd (needed when one thread drives several
 * communicators). */
ncclResult_t ncclGroupStart(void);                                                                  /* nccl.cpp:717 */
ncclResult_t ncclGroupEnd(void);                                                                    /* nccl.cpp:723 */

/* ---- extensions: no counterpart in the reference. They let a GEMM write its result tiles straight into every rank's copy
 * of the matrix (vkzbSetOutputMirrors in vkzb_ext.h), which removes the separate gather altogether. ---- */
/* Collective, blocking on the host, touches no stream: each rank hands in one cudaMalloc'ed buffer; peers[r] receives an
 * address through which this process reaches rank r's buffer (peers[own rank] = buffer). Valid until the communicator goes. */
ncclResult_t vkzbNcclExchangeBuffer(ncclComm_t comm, void* buffer, void** peers);
/* A barrier across the ranks, asynchronous on `stream`: later work on any rank's stream starts only after every rank's
 * stream has reached its barrier (so every earlier write into peer memory has landed). */
ncclResult_t vkzbNcclBarrier(ncclComm_t comm, cudaStream_t stream);

/* Diagnostic: launches the device-side barrier against a peer that does not exist, so its bounded wait (VKZB_NCCL_DEVICE_WAIT_MS,
 * default 20 s) runs out; afterwards ncclCommGetAsyncError reports ncclRemoteError. Nothing faults, the context stays usable.
 * Destroy the communicator afterwards. */
ncclResult_t vkzbNcclSelfTestLostPeer(ncclComm_t comm, cudaStream_t stream);

/* Not served, answering ncclInvalidUsage like the reference's stubs (src/nccl/nccl_stubs.cpp:30-36): ncclCommInitRankScalable,
 * ncclGroupSimulateEnd and the 17 names of nccl_stubs.cpp:11-27. */

#ifdef __cplusplus
}
#endif
#endif /* VKZB_NCCL_H */
