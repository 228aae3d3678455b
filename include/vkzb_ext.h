/*
 * Extensions exported by this repository's libcublas.so.12 beside the cuBLAS names. They have no
 * counterpart in k0zi/Vulkanizer; the closest is its VULKANIZER_LOG=debug line naming the kernel a
 * GEMM was routed to (src/cublas/cublas.cpp:817-820). They exist so tests and the benchmark can prove
 * which hand-written kernel ran, and count launches, without a profiler.
 */
#ifndef VKZB_EXT_H
#define VKZB_EXT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Kernel families a GEMM call can be routed to. */
enum {
    VKZB_PATH_NONE = 0,      /* nothing launched (m, n or batch = 0) */
    VKZB_PATH_SCALE = 1,     /* k = 0: C = beta C */
    VKZB_PATH_GENERIC = 2,   /* CUDA-core tile kernel: any types, leading dimensions, pointer arrays */
    VKZB_PATH_GEMV = 3,      /* m = 1 or n = 1: warp-shuffle HBM-streaming matrix-vector kernel */
    VKZB_PATH_SGEMM = 4,     /* fp32 register-blocked FFMA kernel */
    VKZB_PATH_UMMA = 5,      /* TMA + tcgen05.mma + TMEM kernel (f16, bf16, tf32, int8) */
    VKZB_PATH_DGEMM = 6      /* fp64 DFMA kernel */
};

/* Number of kernels this library has launched in this process since it was loaded. */
uint64_t vkzbLaunchCount(void);
/* VKZB_PATH_* of the most recent GEMM call made on this thread. */
int vkzbLastPath(void);
/*
 * Device-side status word of the tcgen05 kernels for the current device: 0 while every bounded wait
 * (mbarrier phase, TMEM allocation) completed; otherwise a code naming the wait that gave up. Reads
 * the word with a blocking copy, so call it after synchronising the stream. Returns -1 on a CUDA error.
 */
int vkzbDeviceStatus(void);

/*
 * Output mirrors: after this call every GEMM issued through `handle` (cuBLAS or cuBLASLt entry point) whose result matrix
 * lies inside [localBase, localBase + bytes) writes each tile of the result, as it is produced, to the same offset in
 * `count` other buffers as well (at most 7). With the buffers being the other GPUs' copies of the matrix (addresses from
 * vkzbNcclExchangeBuffer of this repository's libnccl.so.2) an N-sharded GEMM leaves the whole matrix on every GPU without
 * a separate all-gather: the NVLink traffic is spread over the GEMM instead of following it.
 * Only the tensor-core kernel with bulk (TMA) stores can do this: D, every mirror, the leading dimension and the column
 * length must be multiples of 16 bytes. A call that cannot honour the mirrors answers CUBLAS_STATUS_NOT_SUPPORTED instead
 * of skipping them. count = 0 switches mirroring off. The caller orders the ranks around the GEMM (vkzbNcclBarrier).
 * Exported by libcublas.so.12 and libcublasLt.so.12 alike (a handle belongs to the library that created it).
 */
int vkzbSetOutputMirrors(void* handle, const void* localBase, size_t bytes, int count, void* const* mirrorBases);

#ifdef __cplusplus
}
#endif
#endif /* VKZB_EXT_H */
