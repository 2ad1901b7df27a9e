// router.cu - the stand-alone MoE routers: softmax top-k (router_top10's contract, src/kernels/cuda/router_top10.cu)
// and sigmoid(+bias) top-k (router_sigmoid.cu:29-74, glm_batch.cu:2063-2100).  One block per token; the arithmetic
// lives in maya_router.cuh.
#include "maya_router.cuh"

namespace maya {
namespace {

constexpr int kRouterThreads = 256;

template<int PER>
__global__ void __launch_bounds__(kRouterThreads) router_softmax_kernel(const float* __restrict__ logits, int n_expert,
                                                                        int k, int* __restrict__ ids,
                                                                        float* __restrict__ weights) {
    extern __shared__ double s_ex[];          // n_expert doubles
    __shared__ RouterShared sh;
    const int t = blockIdx.x, tid = threadIdx.x;
    route_softmax<PER, BlockSync>(logits + (size_t) t * n_expert, n_expert, k, tid, blockDim.x, s_ex, sh);
    if (tid < k) {
        ids[(size_t) t * k + tid] = sh.ids[tid];
        weights[(size_t) t * k + tid] = sh.val[tid];
    }
}

template<int PER>
__global__ void __launch_bounds__(kRouterThreads) router_sigmoid_kernel(const float* __restrict__ logits,
                                                                        const float* __restrict__ bias, int n_expert,
                                                                        int k, float w_scale, int norm_w,
                                                                        int* __restrict__ ids,
                                                                        float* __restrict__ weights) {
    __shared__ RouterShared sh;
    const int t = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    route_sigmoid<PER, BlockSync>(logits + (size_t) t * n_expert, bias, n_expert, k, w_scale, norm_w, tid, nt, sh);
    if (tid < k) {
        ids[(size_t) t * k + tid] = sh.ids[tid];
        weights[(size_t) t * k + tid] = sh.val[tid];
    }
}

int router_threads(int n_expert) {
    int t = n_expert < kRouterThreads ? n_expert : kRouterThreads;
    return (t + 31) & ~31;
}

}  // namespace
}  // namespace maya

using namespace maya;

extern "C" int maya_router_top10(const float* logits, int n_tokens, int n_expert, int k, int* ids, float* weights,
                                 void* stream) {
    if (n_tokens <= 0 || n_expert <= 0 || k <= 0) return MAYA_OK;   // the reference returns without work
    if (!logits || !ids || !weights) return refuse(MAYA_ERR_ARG);
    if (k > 64 || k > n_expert || n_expert > kRouterThreads * kRouterMaxPerThread) return refuse(MAYA_ERR_LIMIT);
    const int nt = router_threads(n_expert);
    const int per = (n_expert + nt - 1) / nt;
    const size_t smem = (size_t) n_expert * sizeof(double);
    cudaStream_t s = as_stream(stream);
    if (per <= 1) router_softmax_kernel<1><<<n_tokens, nt, smem, s>>>(logits, n_expert, k, ids, weights);
    else if (per <= 2) router_softmax_kernel<2><<<n_tokens, nt, smem, s>>>(logits, n_expert, k, ids, weights);
    else if (per <= 4) router_softmax_kernel<4><<<n_tokens, nt, smem, s>>>(logits, n_expert, k, ids, weights);
    else router_softmax_kernel<8><<<n_tokens, nt, smem, s>>>(logits, n_expert, k, ids, weights);
    return note_launch("router_top10");
}

extern "C" int maya_router_sigmoid(const float* logits, const float* bias, int n_tokens, int n_expert, int k,
                                   float w_scale, int norm_w, int* ids, float* weights, void* stream) {
    if (n_tokens <= 0 || n_expert <= 0 || k <= 0) return MAYA_OK;
    if (!logits || !ids || !weights) return refuse(MAYA_ERR_ARG);
    if (k > 64 || k > n_expert || n_expert > kRouterThreads * kRouterMaxPerThread) return refuse(MAYA_ERR_LIMIT);
    const int nt = router_threads(n_expert);
    const int per = (n_expert + nt - 1) / nt;
    cudaStream_t s = as_stream(stream);
    if (per <= 1) router_sigmoid_kernel<1><<<n_tokens, nt, 0, s>>>(logits, bias, n_expert, k, w_scale, norm_w, ids, weights);
    else if (per <= 2) router_sigmoid_kernel<2><<<n_tokens, nt, 0, s>>>(logits, bias, n_expert, k, w_scale, norm_w, ids, weights);
    else if (per <= 4) router_sigmoid_kernel<4><<<n_tokens, nt, 0, s>>>(logits, bias, n_expert, k, w_scale, norm_w, ids, weights);
    else router_sigmoid_kernel<8><<<n_tokens, nt, 0, s>>>(logits, bias, n_expert, k, w_scale, norm_w, ids, weights);
    return note_launch("router_sigmoid");
}
