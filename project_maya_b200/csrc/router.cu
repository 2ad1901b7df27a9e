// router.cu - the MoE routers: softmax top-k (router_top10's contract) and sigmoid(+bias) top-k.
//
// Softmax router, value for value what the reference kernel computes (src/kernels/cuda/router_top10.cu:69-187), so the
// expert ids are bit-exact: float max; exp in double of (double) logit - (double) max; ONE ascending double sum;
// inv = (float) (1 / sum); p = (float) (ex * inv); a stable descending top-k (ties -> lower index); weights
// renormalised in double by max(sum of the k weights, 2^-14).
//
// What differs is only how the selection is carried out: one block per token; p lives in registers, each warp keeps
// its running arg-max and the k rounds cost one shuffle tree plus one shared-memory exchange each.
#include <math.h>

#include "maya_common.cuh"

namespace maya {
namespace {

constexpr int kRouterThreads = 256;
constexpr int kRouterMaxPerThread = 8;   // experts per thread held in registers: n_expert <= 2048 takes this path

// (value, index) arg-max with "greater value, or equal value and lower index" - the stable descending order.
__device__ __forceinline__ void argmax_merge(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

// Selection over scores `sel` (registers, expert e = j * nt + tid), k rounds.  Returns through s_ids / s_val
// (shared, k entries): the chosen ids and the chosen scores' companions `val` (the weights before renormalising).
template<int PER>
__device__ __forceinline__ void select_topk(float (&sel)[PER], const float (&val)[PER], int n_expert, int k, int* s_ids,
                                            float* s_val, float* s_rv, int* s_ri, float* s_rw) {
    const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5, nw = nt >> 5;
    for (int i = 0; i < k; ++i) {
        float bv = -INFINITY, bw = 0.0f;
        int bi = n_expert;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int e = j * nt + tid;
            if (e < n_expert && sel[j] > bv) { bv = sel[j]; bi = e; bw = val[j]; }   // ascending e: lowest index on ties
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            const float ow = __shfl_xor_sync(0xffffffffu, bw, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; bw = ow; }
        }
        if (lane == 0) { s_rv[warp] = bv; s_ri[warp] = bi; s_rw[warp] = bw; }
        __syncthreads();
        float v = s_rv[0], w = s_rw[0];
        int ix = s_ri[0];
        for (int q = 1; q < nw; ++q) {
            const float ov = s_rv[q];
            const int oi = s_ri[q];
            if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; w = s_rw[q]; }
        }
        if (tid == 0 && ix < n_expert) { s_ids[i] = ix; s_val[i] = w; }
        // retire the winner: -inf never beats the -inf start, so it cannot be picked again
#pragma unroll
        for (int j = 0; j < PER; ++j)
            if (j * nt + tid == ix) sel[j] = -INFINITY;
        __syncthreads();
    }
}

template<int PER>
__global__ void __launch_bounds__(kRouterThreads) router_softmax_kernel(const float* __restrict__ logits, int n_expert,
                                                                        int k, int* __restrict__ ids,
                                                                        float* __restrict__ weights) {
    extern __shared__ double s_ex[];          // n_expert doubles
    __shared__ float s_rv[kRouterThreads / 32], s_rw[kRouterThreads / 32];
    __shared__ int s_ri[kRouterThreads / 32];
    __shared__ int s_ids[64];
    __shared__ float s_val[64];
    __shared__ float s_inv;
    const int t = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const float* l = logits + (size_t) t * n_expert;

    float lv[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = j * nt + tid;
        lv[j] = e < n_expert ? l[e] : -INFINITY;
        mx = fmaxf(mx, lv[j]);
    }
    mx = warp_max(mx);
    if ((tid & 31) == 0) s_rv[tid >> 5] = mx;
    __syncthreads();
    mx = s_rv[0];
    for (int q = 1; q < (nt >> 5); ++q) mx = fmaxf(mx, s_rv[q]);
    __syncthreads();

    double ex[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = j * nt + tid;
        ex[j] = e < n_expert ? exp((double) lv[j] - (double) mx) : 0.0;
        if (e < n_expert) s_ex[e] = ex[j];
    }
    __syncthreads();
    if (tid == 0) {
        double sum = 0.0;
        for (int e = 0; e < n_expert; ++e) sum += s_ex[e];   // one thread, ascending: the reference's bits
        s_inv = (float) (1.0 / sum);
    }
    __syncthreads();
    const float inv = s_inv;
    float p[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) p[j] = (j * nt + tid) < n_expert ? (float) (ex[j] * inv) : -INFINITY;
    float sel[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) sel[j] = p[j];
    select_topk<PER>(sel, p, n_expert, k, s_ids, s_val, s_rv, s_ri, s_rw);
    if (tid == 0) {
        double s = 0.0;
        for (int i = 0; i < k; ++i) s += (double) s_val[i];
        const double sc = fmax(s, 6.103515625e-05);   // 2^-14
        for (int i = 0; i < k; ++i) {
            ids[(size_t) t * k + i] = s_ids[i];
            weights[(size_t) t * k + i] = (float) ((double) s_val[i] / sc);
        }
    }
}

template<int PER>
__global__ void __launch_bounds__(kRouterThreads) router_sigmoid_kernel(const float* __restrict__ logits,
                                                                        const float* __restrict__ bias, int n_expert,
                                                                        int k, float w_scale, int norm_w,
                                                                        int* __restrict__ ids,
                                                                        float* __restrict__ weights) {
    __shared__ float s_rv[kRouterThreads / 32], s_rw[kRouterThreads / 32];
    __shared__ int s_ri[kRouterThreads / 32];
    __shared__ int s_ids[64];
    __shared__ float s_val[64];
    const int t = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const float* l = logits + (size_t) t * n_expert;
    float p[PER], sel[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = j * nt + tid;
        if (e < n_expert) {
            p[j] = __fdiv_rn(1.0f, 1.0f + expf(-l[e]));
            sel[j] = bias ? p[j] + bias[e] : p[j];
        } else {
            p[j] = 0.0f;
            sel[j] = -INFINITY;
        }
    }
    select_topk<PER>(sel, p, n_expert, k, s_ids, s_val, s_rv, s_ri, s_rw);
    if (tid == 0) {
        double s = 0.0;
        for (int i = 0; i < k; ++i) s += (double) s_val[i];
        const double sc = fmax(s, 6.103515625e-05);
        for (int i = 0; i < k; ++i) {
            float w = s_val[i];
            if (norm_w) w = (float) ((double) w / sc);
            ids[(size_t) t * k + i] = s_ids[i];
            weights[(size_t) t * k + i] = w * w_scale;
        }
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
