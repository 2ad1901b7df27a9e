// rms_router.cu - the producer in front of the expert FFN: residual add, RMS norm and the router's logits in one launch,
// so that a decode layer is two launches end to end (this one, then the fused layer kernel).
//
// Reference counterparts: glmf::rms_q8 (include/strata/kernels/glm_fast.hpp:534, src/kernels/cuda/glm_fast.cu:5669-5697:
// h += add; x = h * rsqrt(mean(h^2) + eps) * w) and the router job of the multi-GEMV that Glm5Model::fast_moe issues
// next (src/core/glm_fast_path.cu:6925: logits = router_w . x with x in f32; router_w is F32 or BF16).  The q8_1 image
// of x that rms_q8 also writes is made by the layer kernel itself here.
//
// Every block recomputes the norm of the (small) hidden state - no grid-wide step - and then owns a slice of the
// experts' router rows; block 0 also writes x and the updated residual stream.  The residual goes to h_out, which must
// not alias h when add is given (other blocks may still be reading h).
#include "maya_common.cuh"

namespace maya {
namespace {

constexpr int kRmsThreads = 256;

__global__ void __launch_bounds__(kRmsThreads) rms_router_kernel(const float* __restrict__ h, const float* __restrict__ add,
                                                                 const float* __restrict__ w, float eps, int n,
                                                                 const void* __restrict__ router, int router_is_bf16, int n_expert,
                                                                 float* __restrict__ h_out, float* __restrict__ x_out,
                                                                 float* __restrict__ logits) {
    extern __shared__ __align__(16) float xs[];
    __shared__ float sred[kRmsThreads / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float ss = 0.0f;
    for (int e = tid; e < n; e += kRmsThreads) {
        float t = h[e];
        if (add != nullptr) t += add[e];
        xs[e] = t;
        ss += t * t;
    }
    ss = warp_sum(ss);
    if (lane == 0) sred[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kRmsThreads / 32; ++i) tot += sred[i];
    const float inv = rsqrtf(tot / (float) n + eps);
    for (int e = tid; e < n; e += kRmsThreads) {
        const float t = xs[e], xv = t * inv * w[e];
        xs[e] = xv;
        if (blockIdx.x == 0) {
            x_out[e] = xv;
            if (h_out != nullptr) h_out[e] = t;
        }
    }
    __syncthreads();
    // router rows: a warp per expert, lanes stride the row
    for (int ex = blockIdx.x * (kRmsThreads / 32) + warp; ex < n_expert; ex += gridDim.x * (kRmsThreads / 32)) {
        float acc = 0.0f;
        if (router_is_bf16) {
            const uint16_t* r = (const uint16_t*) router + (size_t) ex * n;
            for (int e = lane; e < n; e += 32) acc = __fmaf_rn(__uint_as_float((uint32_t) r[e] << 16), xs[e], acc);
        } else {
            const float* r = (const float*) router + (size_t) ex * n;
            for (int e = lane; e < n; e += 32) acc = __fmaf_rn(r[e], xs[e], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) logits[ex] = acc;
    }
}

}  // namespace
}  // namespace maya

using namespace maya;

extern "C" int maya_rms_router(const float* h, const float* add, const float* norm_w, float eps, int n_embd,
                               const void* router_w, int router_is_bf16, int n_expert, float* h_out, float* x_out,
                               float* logits, void* stream) {
    if (!h || !norm_w || !router_w || !x_out || !logits || n_embd <= 0 || n_expert <= 0) return refuse(MAYA_ERR_ARG);
    if (add != nullptr && h_out == h) return refuse(MAYA_ERR_ARG);       // other blocks still read h
    const size_t smem = (size_t) n_embd * sizeof(float);
    if (smem > 200 * 1024) return refuse(MAYA_ERR_LIMIT);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(rms_router_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess)
        return note_launch("rms_router smem attribute");
    const int blocks = (n_expert + kRmsThreads / 32 - 1) / (kRmsThreads / 32);
    rms_router_kernel<<<blocks, kRmsThreads, smem, as_stream(stream)>>>(h, add, norm_w, eps, n_embd, router_w, router_is_bf16,
                                                                        n_expert, h_out, x_out, logits);
    return note_launch("rms_router");
}
