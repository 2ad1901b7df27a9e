// quantize_q8_1.cu - f32 / bf16 activations -> q8_1 blocks, and SwiGLU -> q8_1 (the shared expert's h).
//
// Arithmetic of the reference quantizer (src/kernels/cuda/native_mmvq.cu:140-152, iq_kernels.cu:639-654,
// glm_fast.cu:165-174): per 32 values d = min(amax / 127, 65504), q = round(x / d) clamped to +-127, the block keeps
// {f16 d, f16 sum of the original values}.  One warp per block, IEEE division.
#include "maya_common.cuh"

namespace maya {
namespace {

template<bool BF16>
__global__ void __launch_bounds__(256) quantize_q8_1_kernel(const void* __restrict__ x, uint8_t* __restrict__ y,
                                                            int64_t n_blocks) {
    const int lane = threadIdx.x & 31;
    const int64_t b = (int64_t) blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= n_blocks) return;
    float v;
    if (BF16) v = __uint_as_float((uint32_t) ((const uint16_t*) x)[b * 32 + lane] << 16);
    else v = ((const float*) x)[b * 32 + lane];
    q8_1_store_warp(v, y + b * kQ81Bytes, lane);
}

__global__ void __launch_bounds__(256) swiglu_q8_1_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                                          float limit, int64_t n_blocks, uint8_t* __restrict__ hq) {
    const int lane = threadIdx.x & 31;
    const int64_t b = (int64_t) blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= n_blocks) return;
    q8_1_store_warp(swiglu(gate[b * 32 + lane], up[b * 32 + lane], limit), hq + b * kQ81Bytes, lane);
}

}  // namespace
}  // namespace maya

using namespace maya;

static int quantize_any(const void* x, void* xq, int n_in, int ncols, void* stream, bool bf16) {
    if (ncols <= 0) return MAYA_OK;
    if (!x || !xq || n_in <= 0 || n_in % 32) return refuse(MAYA_ERR_ARG);
    const int64_t nb = (int64_t) ncols * (n_in / 32);
    const unsigned grid = (unsigned) ((nb + 7) / 8);
    if (bf16) quantize_q8_1_kernel<true><<<grid, 256, 0, as_stream(stream)>>>(x, (uint8_t*) xq, nb);
    else quantize_q8_1_kernel<false><<<grid, 256, 0, as_stream(stream)>>>(x, (uint8_t*) xq, nb);
    return note_launch("quantize_q8_1");
}

extern "C" int maya_quantize_q8_1(const float* x, void* xq, int n_in, int ncols, void* stream) {
    return quantize_any(x, xq, n_in, ncols, stream, false);
}
extern "C" int maya_quantize_q8_1_bf16(const uint16_t* x, void* xq, int n_in, int ncols, void* stream) {
    return quantize_any(x, xq, n_in, ncols, stream, true);
}
extern "C" int maya_swiglu_q8_1(const float* gate, const float* up, float limit, int64_t n, void* hq, void* stream) {
    if (n <= 0) return MAYA_OK;
    if (!gate || !up || !hq || n % 32) return refuse(MAYA_ERR_ARG);
    const int64_t nb = n / 32;
    swiglu_q8_1_kernel<<<(unsigned) ((nb + 7) / 8), 256, 0, as_stream(stream)>>>(gate, up, limit, nb, (uint8_t*) hq);
    return note_launch("swiglu_q8_1");
}
