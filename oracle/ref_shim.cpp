// TEST INFRASTRUCTURE. C entry points around k0zi/Vulkanizer's own CPU GEMM, so that tests and the benchmark's
// CPU baseline can call the reference's code for this path through ctypes. This file contains no arithmetic:
// it forwards to vulkanizer::npu::createCpuBackend()->gemm (src/npu/backend.cpp:28-52, single-threaded) and to
// the staged pipeline stage -> packTransposed -> hostGemm -> epilogue (src/npu/backend.cpp:58-78,
// src/npu/host.cpp:114-235, hostGemm multi-threaded over result rows), both compiled from the reference's
// sources where they lie by oracle/Makefile into oracle/_ref/libvkref.so.
#include <cstdint>
#include <memory>
#include <thread>

#include "npu/host.h"
#include "npu/npu.h"

using namespace vulkanizer::npu;

static DType dtype(int code) { return code == 1 ? DType::F16 : code == 2 ? DType::BF16 : DType::F32; }

static Backend* cpuBackend() {
    static std::unique_ptr<Backend> b = createCpuBackend();
    return b.get();
}

extern "C" {

// Type codes: 0 f32, 1 f16, 2 bf16. Returns 1 on success.
int vkref_cpu_gemm(int transA, int transB, int64_t m, int64_t n, int64_t k, int64_t batch, float alpha, const void* A, int typeA,
                   int64_t lda, int64_t strideA, const void* B, int typeB, int64_t ldb, int64_t strideB, float beta, void* C,
                   int typeC, int64_t ldc, int64_t strideC) {
    GemmArgs g;
    g.shape.transA = transA != 0, g.shape.transB = transB != 0;
    g.shape.m = m, g.shape.n = n, g.shape.k = k, g.shape.batch = batch;
    g.shape.a = dtype(typeA), g.shape.b = dtype(typeB), g.shape.c = dtype(typeC);
    g.alpha = alpha, g.beta = beta;
    g.a = A, g.lda = lda, g.strideA = strideA;
    g.b = B, g.ldb = ldb, g.strideB = strideB;
    g.c = C, g.ldc = ldc, g.strideC = strideC;
    return cpuBackend()->gemm(g) ? 1 : 0;
}

// The multi-threaded path, one batch entry: pack op(B)^T and op(A)^T into the backend's staging buffers,
// hostGemm on all cores, epilogue into C. Returns the number of threads hostGemm used, 0 on failure.
int vkref_staged_gemm(int transA, int transB, int64_t m, int64_t n, int64_t k, float alpha, const void* A, int typeA, int64_t lda,
                      const void* B, int typeB, int64_t ldb, float beta, void* C, int typeC, int64_t ldc) {
    GemmShape s;
    s.transA = transA != 0, s.transB = transB != 0;
    s.m = m, s.n = n, s.k = k, s.batch = 1;
    s.a = dtype(typeA), s.b = dtype(typeB), s.c = dtype(typeC);
    Staging st;
    Backend* b = cpuBackend();
    if (!b->stage(s, st)) return 0;
    // lhs = op(B)^T (n x k), rhs = op(A)^T (k x m), result n x m, all row-major (src/npu/host.h:3-6)
    packTransposed(B, s.b, ldb, s.transB, k, n, st.lhs, st.in, st.k);
    packTransposed(A, s.a, lda, s.transA, m, k, st.rhs, st.in, st.n);
    if (!b->runStaged(st)) return 0;
    epilogue(st.result, st.out, st.n, alpha, beta, C, s.c, ldc, m, n);
    const int64_t hw = std::thread::hardware_concurrency();
    int64_t threads = hw < (m * n * k >> 20) ? hw : (m * n * k >> 20);
    if (threads < 1) threads = 1;
    if (threads > st.m) threads = st.m;
    return int(threads);
}

uint16_t vkref_float_to_half(float f) { return floatToHalf(f); }
float vkref_half_to_float(uint16_t h) { return halfToFloat(h); }
uint16_t vkref_float_to_bf16(float f) { return floatToBf16(f); }
float vkref_bf16_to_float(uint16_t h) { return bf16ToFloat(h); }
int vkref_hardware_threads(void) { return int(std::thread::hardware_concurrency()); }

}  // extern "C"
