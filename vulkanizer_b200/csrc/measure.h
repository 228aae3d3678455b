// Measurement switches. The shipped libraries are built WITHOUT VKZB_MEASURE: every switch then folds to its default at
// compile time and no environment variable can change which kernel variant a GEMM call takes. `make MEASURE=1` builds
// libraries whose tile shape, pairing, split and similar choices can be forced from the environment, for experiments.
#pragma once

#include <cstdlib>

namespace vkzb {

#ifdef VKZB_MEASURE
inline int measureKnob(const char* name, int fallback) {
    const char* v = std::getenv(name);
    return v ? std::atoi(v) : fallback;
}
#else
constexpr int measureKnob(const char*, int fallback) { return fallback; }
#endif

}  // namespace vkzb
