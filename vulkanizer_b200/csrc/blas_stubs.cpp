// cuBLAS names that programs link against but this library does not implement (complex and BLAS 1/2 routines,
// batched factorizations and triangular solves, the "_64" forms of those). Like k0zi/Vulkanizer's
// src/cublas/cublas_stubs.cpp:241-247, each is a parameterless C function (the C calling convention lets it
// ignore its arguments) that answers CUBLAS_STATUS_NOT_SUPPORTED, with a one-time note on stderr.
// The names come from blas_stub_names.def, one per line.
#include <atomic>
#include <cstdio>

namespace {
int unimplemented(const char* name, std::atomic<bool>& told) {
    if (!told.exchange(true)) std::fprintf(stderr, "vkzb: %s is not implemented (CUBLAS_STATUS_NOT_SUPPORTED)\n", name);
    return 15;  // CUBLAS_STATUS_NOT_SUPPORTED
}
}  // namespace

#define VKZB_STUB(name)                         \
    extern "C" int name() {                     \
        static std::atomic<bool> told{false};   \
        return unimplemented(#name, told);      \
    }
#include "blas_stub_list.inc"
