// ref_shim_q8k.cpp - TEST INFRASTRUCTURE.  The reference's host transcription of ggml's Q8_K activation quantizer
// (src/kernels/quantize_act_parity.cpp:139-176, file-local), reached the same way as ref_shim_router.cpp does.
#define main static __attribute__((unused)) maya_ref_unused_main
#include "src/kernels/quantize_act_parity.cpp"
#undef main

extern "C" __attribute__((visibility("default")))
void ref_quantize_q8_K(const float* x, long long n, unsigned char* blocks) {
    std::vector<uint8_t> b;
    std::vector<float> back;
    reference_q8_K(x, n, b, back, -127.0f);
    std::memcpy(blocks, b.data(), b.size());
}
