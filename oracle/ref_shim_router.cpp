// ref_shim_router.cpp - TEST INFRASTRUCTURE.  Reaches the host reference inside the reference's own router test
// (src/kernels/router_top10_parity.cpp:36-60, a file-local function) by compiling that file, where it lies, as part
// of this translation unit with its main() turned into an unused static function.  Built only where the reference
// tree is present; the output goes to oracle/_ref/.
#define main static __attribute__((unused)) maya_ref_unused_main
#include "src/kernels/router_top10_parity.cpp"
#undef main

extern "C" __attribute__((visibility("default")))
void ref_router_reference(const float* logits, int n_tokens, int n_expert, int k, int* ids, float* w) {
    for (int t = 0; t < n_tokens; ++t)
        reference(logits + (size_t) t * n_expert, n_expert, k, ids + (size_t) t * k, w + (size_t) t * k);
}

// The four input distributions of the reference's test, from its generator and seed
// (router_top10_parity.cpp:119-146: mt19937(2024), normal(0, 1), 64 tokens x 512 experts).  out: 4 * 64 * 512 floats.
extern "C" __attribute__((visibility("default")))
void ref_router_test_inputs(float* out) {
    const int NE = 512, NT = 64;
    std::mt19937 rng(2024);
    std::normal_distribution<float> gauss(0.0f, 1.0f);
    float* a = out;
    float* b = out + (size_t) NT * NE;
    float* c = b + (size_t) NT * NE;
    float* d = c + (size_t) NT * NE;
    for (int i = 0; i < NT * NE; ++i) a[i] = gauss(rng);
    for (int i = 0; i < NT * NE; ++i) b[i] = 0.5f;
    for (int t = 0; t < NT; ++t)
        for (int e = 0; e < NE; ++e) c[(size_t) t * NE + e] = (e < 12) ? 2.0f : gauss(rng);
    for (int i = 0; i < NT * NE; ++i) d[i] = 0.0f;
    for (int t = 0; t < NT; ++t) d[(size_t) t * NE + (t % NE)] = 20.0f;
}
