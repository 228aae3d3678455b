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

// Derivative of geluTanh.
__device__ __forceinline__ float geluTanhGrad(float x) {
    const float u = 0.7978845608f * (x + 0.044715f * x * x * x);
    const float t = tanhf(u);
    return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * 0.7978845608f * (1.0f + 3.0f * 0.044715f * x * x);
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
//
// Kernels call store() once per result from fully unrolled loops, so its inlined body must stay a handful of
// instructions or the unrolled code outgrows the instruction cache (measured: a 128 x 256 tile took 34 us to
// write with the whole type switch inlined 32 times over, against under 2 us of arithmetic). The common cases,
// a plain f32 / f16 / bf16 / s32 store with or without beta * C of the same type, are inlined; everything else
// (mixed C and D types, bias, activation, the extra rounding) goes through one out-of-line function.
enum StoreMode : int { kStoreSlow = 0, kStoreF32 = 1, kStoreF16 = 2, kStoreBF16 = 3, kStoreS32 = 4, kStoreF64 = 5 };

template <typename Acc>
struct Epilogue {
    char* D;
    const char* C;
    const char* bias;
    char* aux;
    long long ldd, ldc, auxLd;
    Acc alpha, beta;
    int typeD, typeC, typeBias, activation, roundBeforeBias, biasAlongN, typeAux, auxMode;
    int mode;       // StoreMode
    int typedMode;  // the StoreMode D and C alone ask for: what `mode` would be without bias, activation and the extra rounding
    bool readC;
    bool post;      // bias, activation or the extra rounding follow alpha * acc + beta * C

    __device__ __forceinline__ void init(const EpilogueArgs& e, long long batchEntry) {
        const double a = readScalar(e.scalars.alphaDev, e.scalars.alphaHost, e.scalars.type);
        const double b = readScalar(e.scalars.betaDev, e.scalars.betaHost, e.scalars.type);
        alpha = Acc(a);
        beta = Acc(b);
        readC = b != 0.0;  // beta = 0: C is not read, so NaNs in it do not propagate (gemm.comp:143)
        typeD = e.typeD, typeC = e.typeC, typeBias = e.typeBias;
        activation = e.activation, roundBeforeBias = e.roundBeforeBias;
        biasAlongN = e.biasAlongN, typeAux = e.typeAux, auxMode = e.auxMode, auxLd = e.auxLd;
        ldd = e.ldd, ldc = e.ldc;
        if (e.pointerArrays) {
            D = static_cast<char*>(static_cast<void* const*>(e.D)[batchEntry]);
            C = D;
        } else {
            D = static_cast<char*>(e.D) + batchEntry * e.strideD * dtypeSize(e.typeD);
            C = static_cast<const char*>(e.C) + batchEntry * e.strideC * dtypeSize(e.typeC);
        }
        bias = e.bias ? static_cast<const char*>(e.bias) + batchEntry * e.biasStride * dtypeSize(e.typeBias) : nullptr;
        aux = nullptr;
        if (e.aux && e.auxMode != kAuxNone) {
            const bool mask = e.auxMode == kAuxWriteMask || e.auxMode == kAuxReadMask;  // strides of a mask count bits
            aux = static_cast<char*>(e.aux) + (mask ? batchEntry * e.auxStride / 8 : batchEntry * e.auxStride * dtypeSize(e.typeAux));
        }
        post = bias || activation != kActNone || roundBeforeBias || aux;
        const bool mixed = readC && typeC != typeD;
        if constexpr (std::is_same_v<Acc, double>) typedMode = kStoreF64;
        else if constexpr (std::is_same_v<Acc, int>) typedMode = typeD == kS32 && !mixed ? kStoreS32 : kStoreSlow;
        else typedMode = mixed ? kStoreSlow : typeD == kF32 ? kStoreF32 : typeD == kF16 ? kStoreF16 : typeD == kBF16 ? kStoreBF16 : kStoreSlow;
        mode = post && !std::is_same_v<Acc, double> ? kStoreSlow : typedMode;
    }

    // What follows alpha * acc + beta * C when `post` is set and no auxiliary matrix is involved (float accumulators).
    __device__ __forceinline__ float finish(float v, float biasValue) const {
        if (roundBeforeBias) v = roundTo(v, typeD);
        v += biasValue;
        if (activation == kActRelu) v = fmaxf(v, 0.0f);
        else if (activation == kActGelu) v = geluTanh(v);
        return v;
    }

    __device__ __forceinline__ float biasAt(int row, int col) const { return bias ? loadAs<float>(bias, biasAlongN ? col : row, typeBias) : 0.0f; }

    // The same for one result at (row, col) with the auxiliary matrix handled by this thread alone: the mask bit is set or
    // cleared with an atomic on its 32-bit word, so any assignment of results to threads is safe (the tensor-core kernel has a
    // faster form that writes whole words, one per warp and column).
    __device__ __noinline__ float finishAt(float v, int row, int col) const {
        if (roundBeforeBias) v = roundTo(v, typeD);
        v += biasAt(row, col);
        const long long at = row + col * auxLd;
        if (auxMode == kAuxWriteInput) storeFloat(aux, at, typeAux, v);
        if (auxMode == kAuxWriteMask) {
            unsigned* word = reinterpret_cast<unsigned*>(aux) + (at >> 5);
            const unsigned bit = 1u << (at & 31);
            if (v > 0.0f) atomicOr(word, bit);
            else atomicAnd(word, ~bit);
        }
        if (activation == kActRelu) v = fmaxf(v, 0.0f);
        else if (activation == kActGelu) v = geluTanh(v);
        else if (activation == kActDRelu) v = (reinterpret_cast<const unsigned*>(aux)[at >> 5] >> (at & 31)) & 1u ? v : 0.0f;
        else if (activation == kActDGelu) v *= geluTanhGrad(loadAs<float>(aux, at, typeAux));
        return v;
    }

    // The general form: any C / D / bias types, bias, activation.
    __device__ __noinline__ void storeSlow(int row, int col, Acc acc) const {
        const long long di = row + col * ldd;
        if constexpr (std::is_same_v<Acc, int>) {
            int v = alpha * acc;
            if (readC) v += beta * loadAs<int>(C, row + col * ldc, typeC);
            if (typeD == kS32) static_cast<int*>(static_cast<void*>(D))[di] = v;
            else storeFloat(D, di, typeD, float(v));
        } else if constexpr (std::is_same_v<Acc, float>) {
            float v = alpha * acc;
            if (readC) v += beta * loadAs<float>(C, row + col * ldc, typeC);
            if (aux) {
                v = finishAt(v, row, col);
            } else {
                if (roundBeforeBias) v = roundTo(v, typeD);
                v += biasAt(row, col);
                if (activation == kActRelu) v = fmaxf(v, 0.0f);
                else if (activation == kActGelu) v = geluTanh(v);
            }
            storeFloat(D, di, typeD, v);
        }
    }

    // One result, storage type fixed at compile time (MODE is a StoreMode other than kStoreSlow).
    template <int MODE>
    __device__ __forceinline__ void storeAs(int row, int col, Acc acc) const {
        const long long di = row + col * ldd, ci = row + col * ldc;
        if constexpr (MODE == kStoreF64) {
            double v = alpha * acc;
            if (readC) v += beta * reinterpret_cast<const double*>(C)[ci];
            reinterpret_cast<double*>(D)[di] = v;
        } else if constexpr (MODE == kStoreS32) {
            int v = alpha * acc;
            if (readC) v += beta * reinterpret_cast<const int*>(C)[ci];
            reinterpret_cast<int*>(D)[di] = v;
        } else if constexpr (MODE == kStoreF32) {
            float v = alpha * acc;
            if (readC) v += beta * reinterpret_cast<const float*>(C)[ci];
            reinterpret_cast<float*>(D)[di] = v;
        } else if constexpr (MODE == kStoreF16) {
            float v = alpha * acc;
            if (readC) v += beta * __half2float(reinterpret_cast<const __half*>(C)[ci]);
            reinterpret_cast<__half*>(D)[di] = __float2half_rn(v);
        } else {
            float v = alpha * acc;
            if (readC) v += beta * __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(C)[ci]);
            reinterpret_cast<__nv_bfloat16*>(D)[di] = __float2bfloat16_rn(v);
        }
    }

    // For kernels with few results per thread: the plain fp32 (or s32 / f64) store inline, the rest out of line.
    __device__ __forceinline__ void store(int row, int col, Acc acc) const {
        if constexpr (std::is_same_v<Acc, double>) {
            storeAs<kStoreF64>(row, col, acc);
        } else if constexpr (std::is_same_v<Acc, int>) {
            if (mode == kStoreS32) storeAs<kStoreS32>(row, col, acc);
            else storeSlow(row, col, acc);
        } else {
            if (mode == kStoreF32) storeAs<kStoreF32>(row, col, acc);
            else if (mode == kStoreF16) storeAs<kStoreF16>(row, col, acc);
            else if (mode == kStoreBF16) storeAs<kStoreBF16>(row, col, acc);
            else storeSlow(row, col, acc);
        }
    }
};

}  // namespace vkzb
