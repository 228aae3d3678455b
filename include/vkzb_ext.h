/*
 * Extensions exported by this repository's libcublas.so.12 beside the cuBLAS names. They have no
 * counterpart in k0zi/Vulkanizer; the closest is its VULKANIZER_LOG=debug line naming the kernel a
 * GEMM was routed to (src/cublas/cublas.cpp:817-820). They exist so tests and the benchmark can prove
 * which hand-written kernel ran, and count launches, without a profiler.
 */
#ifndef VKZB_EXT_H
#define VKZB_EXT_H

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

#ifdef __cplusplus
}
#endif
#endif /* VKZB_EXT_H */
