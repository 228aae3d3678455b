// Device-side helpers every kernel family shares: typed loads and stores with one round-to-nearest-even
// conversion at the store (as k0zi/Vulkanizer's shaders do, src/cublas/shaders/gemm.comp:45-74), alpha and
// beta in either pointer mode, and the fused epilogue D = act(alpha * acc + beta * C + bias) that replaces
// the reference's separate pass over D (src/cublas/shaders/epilogue.comp:73-91).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "gemm_problem.h"

namespace vkzb {

template <typename T>
__device__ __forceinline__ T loadAs(const void* base, long long index, int type);

template <>
__device__ __forceinline__ float loadAs<float>(const void* base, long long index, int type) {
    switch (type) {
    case kF32: return static_cast<const float*>(base)[index];
    case kF16: return __half2float(static_cast<const __half*>(base)[index]);
    case kBF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[index]);
    case kS8: return float(static_cast<const signed char*>(base)[index]);
    case kS32: return float(static_cast<const int*>(base)[index]);
    default: return float(static_cast<const double*>(base)[index]);
    }
}

template <>
__device__ __forceinline__ double loadAs<double>(const void* base, long long index, int type) {
    if (type == kF64) return static_cast<const double*>(base)[index];
    return double(loadAs<float>(base, index, type));
}

template <>
__device__ __forceinline__ int loadAs<int>(const void* base, long long index, int type) {
    if (type == kS8) return int(static_cast<const signed char*>(base)[index]);
    if (type == kS32) return static_cast<const int*>(base)[index];
    return int(loadAs<float>(base, index, type));
}

__device__ __forceinline__ void storeFloat(void* base, long long index, int type, float v) {
    switch (type) {
    case kF32: static_cast<float*>(base)[index] = v; break;
    case kF16: static_cast<__half*>(base)[index] = __float2half_rn(v); break;
    case kBF16: static_cast<__nv_bfloat16*>(base)[index] = __float2bfloat16_rn(v); break;
    default: break;
    }
}

__device__ __forceinline__ float roundTo(float v, int type) {
    if (type == kF16) return __half2float(__float2half_rn(v));
    if (type == kBF16) return __bfloat162float(__float2bfloat16_rn(v));
    return v;
}

// tanh-GELU with the constants of the reference's epilogue shader (epilogue.comp:86-89).
__device__ __forceinline__ float geluTanh(float x) {
    return 0.5f * x * (1.0f + tanhf(0.7978845608f * (x + 0.044715f * x * x * x)));
}

__device__ __forceinline__ double readScalar(const void* dev, double host, int type) {
    if (!dev) return host;
    switch (type) {
    case kScalarF16: return double(__half2float(*static_cast<const __half*>(dev)));
    case kScalarS32: return double(*static_cast<const int*>(dev));
    case kScalarF64: return *static_cast<const double*>(dev);
    default: return double(*static_cast<const float*>(dev));
    }
}

// Per-thread view of the epilogue for one batch entry. Acc is float, int or double.
template <typename Acc>
struct Epilogue {
    char* D;
    const char* C;
    const char* bias;
    long long ldd, ldc;
    Acc alpha, beta;
    int typeD, typeC, typeBias, activation, roundBeforeBias;
    bool readC;

    __device__ __forceinline__ void init(const EpilogueArgs& e, long long batchEntry) {
        const double a = readScalar(e.scalars.alphaDev, e.scalars.alphaHost, e.scalars.type);
        const double b = readScalar(e.scalars.betaDev, e.scalars.betaHost, e.scalars.type);
        alpha = Acc(a);
        beta = Acc(b);
        readC = b != 0.0;  // beta = 0: C is not read, so NaNs in it do not propagate (gemm.comp:143)
        typeD = e.typeD, typeC = e.typeC, typeBias = e.typeBias;
        activation = e.activation, roundBeforeBias = e.roundBeforeBias;
        ldd = e.ldd, ldc = e.ldc;
        if (e.pointerArrays) {
            D = static_cast<char*>(static_cast<void* const*>(e.D)[batchEntry]);
            C = D;
        } else {
            D = static_cast<char*>(e.D) + batchEntry * e.strideD * dtypeSize(e.typeD);
            C = static_cast<const char*>(e.C) + batchEntry * e.strideC * dtypeSize(e.typeC);
        }
        bias = e.bias ? static_cast<const char*>(e.bias) + batchEntry * e.biasStride * dtypeSize(e.typeBias) : nullptr;
    }

    __device__ __forceinline__ void store(int row, int col, Acc acc) const {
        const long long di = row + col * ldd;
        if constexpr (std::is_same_v<Acc, double>) {
            double v = alpha * acc;
            if (readC) v += beta * static_cast<const double*>(static_cast<const void*>(C))[row + col * ldc];
            static_cast<double*>(static_cast<void*>(D))[di] = v;
        } else if constexpr (std::is_same_v<Acc, int>) {
            int v = alpha * acc;
            if (readC) v += beta * loadAs<int>(C, row + col * ldc, typeC);
            if (typeD == kS32) static_cast<int*>(static_cast<void*>(D))[di] = v;
            else storeFloat(D, di, typeD, float(v));
        } else {
            float v = alpha * acc;
            if (readC) v += beta * loadAs<float>(C, row + col * ldc, typeC);
            if (roundBeforeBias) v = roundTo(v, typeD);
            if (bias) v += loadAs<float>(bias, row, typeBias);
            if (activation == kActRelu) v = fmaxf(v, 0.0f);
            else if (activation == kActGelu) v = geluTanh(v);
            storeFloat(D, di, typeD, v);
        }
    }
};

}  // namespace vkzb
