// TEST INFRASTRUCTURE.  The reference's tests draw their inputs with std::mt19937 + std::normal_distribution<float>
// (src/models/deepseek41/kernels/test_util.hpp:88-94, tests/kernels/native_expert_parity.cpp:69-72), whose output depends on
// the C++ standard library; this reproduces those streams with libstdc++ so that frozen hashes of the reference's tests
// can be re-derived from the same inputs.
#include <cstddef>
#include <cstdint>
#include <random>

extern "C" __attribute__((visibility("default"))) void std_randn(float* out, size_t n, uint32_t seed, float sigma, float mean) {
    std::mt19937 g(seed);
    std::normal_distribution<float> d(mean, sigma);
    for (size_t i = 0; i < n; ++i) out[i] = d(g);
}
