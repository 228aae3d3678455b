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

#ifndef VKZB_HAVE_CUDA_TYPES
typedef struct CUstream_st* cudaStream_t;
#endif

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
 * How the most recent tensor-core (VKZB_PATH_UMMA) launch made on this thread was laid out: bits 0-9 the tile's column count
 * (64, 128 or 256), bit 10 two-CTA pairs (tiles of 256 rows), bit 11 the wide-epilogue variant, bits 12-15 the number of
 * splits along k (1: none).
 */
int vkzbLastPlan(void);
/*
 * Device-side status word of the tcgen05 and matrix-vector kernels for the current device: 0 while every bounded
 * wait (mbarrier phase, TMEM allocation) completed; otherwise a code naming the wait that gave up (1-4: tcgen05
 * kernel roles, 16: a bulk copy of the matrix-vector kernel). Reads
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

/*
 * cublasSgemm for callers that may not allocate device memory. No counterpart in the reference.
 *
 * Who needs it: a process that gives all device memory to its own pool at start-up, or that is in a phase where cudaMalloc
 * is unacceptable because it synchronises the device. A handle of this library allocates the scratch memory of its split-k
 * kernels at the first call that splits, which such a caller cannot allow; this entry point takes no handle and runs the same
 * split-k FFMA kernel on a scratch array built into the library image. It calls no cudaMalloc, cudaFree or other allocating
 * routine (a test compares the driver's free-memory figure before and after).
 *
 * C = alpha op(A) op(B) + beta C, fp32, column-major, alpha and beta on the host, asynchronous on `stream`; transa / transb
 * are cublasOperation_t values; the return value is a cublasStatus_t value.
 * Limit: the built-in array holds 4096 counters and 4 MiB of partial tiles, enough for results of up to 256 tiles of
 * 64 x 64 (m * n up to about 2^20, e.g. 1024 x 1024); k is cut into up to 8 slices as far as that room allows. A larger
 * result is refused with CUBLAS_STATUS_INVALID_VALUE and a line on stderr; k = 0 and matrix-vector shapes answer
 * CUBLAS_STATUS_NOT_SUPPORTED (use the handle-based entry points for those).
 * First call: the first call on each device (with that device current) asks the runtime for the array's device address. That
 * makes the driver load the array's module onto the device, which is when its memory is reserved and which may synchronise the
 * device, so make one call per device during start-up, and before starting any stream capture. Later calls do no set-up.
 * Sharing: every call on a device uses the one array, which keeps what the last call left in it (each call clears the
 * counters it is about to use, in stream order): two calls that overlap on the GPU would corrupt each other, so issue them on
 * one stream or order them yourself. Only libcublas.so.12 carries the array (libcublasLt.so.12 does not), so a GPU holds one
 * copy, 4 MiB + 16 KiB, from the first call until the process ends.
 */
int vkzbSgemmStaticScratch(cudaStream_t stream, int transa, int transb, int m, int n, int k, const float* alpha, const float* A,
                           int lda, const float* B, int ldb, const float* beta, float* C, int ldc);

#ifdef __cplusplus
}
#endif
#endif /* VKZB_EXT_H */
