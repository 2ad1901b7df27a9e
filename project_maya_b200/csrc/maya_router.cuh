// maya_router.cuh - the routers' device code, shared by the stand-alone router kernels and the fused decode layer.
//
// Softmax router, value for value what the reference kernel computes (src/kernels/cuda/router_top10.cu:69-187), so the
// expert ids are bit-exact: float max; exp in double of (double) logit - (double) max; ONE ascending double sum;
// inv = (float) (1 / sum); p = (float) (ex * inv); a stable descending top-k (ties -> lower index); weights
// renormalised in double by max(sum of the k weights, 2^-14).
//
// What differs is only how the selection is carried out: one thread group per token; p lives in registers, each warp
// keeps its running arg-max and the k rounds cost one shuffle tree plus one shared-memory exchange each.
//
// The thread group is `nt` threads (a multiple of 32) that synchronise through `Sync::sync()`: the whole block
// (__syncthreads) or a named barrier when only part of a block routes.
#pragma once

#include <math.h>

#include "maya_common.cuh"

namespace maya {

constexpr int kRouterMaxWarps = 8;        // threads per routing group <= 256
constexpr int kRouterMaxPerThread = 8;    // experts per thread held in registers: n_expert <= 2048

struct BlockSync {
    __device__ __forceinline__ static void sync() { __syncthreads(); }
};
template<int ID, int N> struct NamedSync {
    __device__ __forceinline__ static void sync() { asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(N) : "memory"); }
};

struct RouterShared {
    float rv[kRouterMaxWarps], rw[kRouterMaxWarps];
    int ri[kRouterMaxWarps];
    int ids[64];
    float val[64];
    float inv;
};

// k rounds of arg-max over `sel` (expert e = j * nt + tid), "greater value, or equal value and lower index" - the
// stable descending order.  The chosen ids and their companions `val` land in sh.ids / sh.val.
template<int PER, class Sync>
__device__ __forceinline__ void select_topk(float (&sel)[PER], const float (&val)[PER], int n_expert, int k, int tid,
                                            int nt, RouterShared& sh) {
    const int lane = tid & 31, warp = tid >> 5, nw = nt >> 5;
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
        if (lane == 0) { sh.rv[warp] = bv; sh.ri[warp] = bi; sh.rw[warp] = bw; }
        Sync::sync();
        float v = sh.rv[0], w = sh.rw[0];
        int ix = sh.ri[0];
        for (int q = 1; q < nw; ++q) {
            const float ov = sh.rv[q];
            const int oi = sh.ri[q];
            if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; w = sh.rw[q]; }
        }
        if (tid == 0 && ix < n_expert) { sh.ids[i] = ix; sh.val[i] = w; }
        // retire the winner: -inf never beats the -inf start, so it cannot be picked again
#pragma unroll
        for (int j = 0; j < PER; ++j)
            if (j * nt + tid == ix) sel[j] = -INFINITY;
        Sync::sync();
    }
}

// One token's softmax routing by the calling thread group.  l: n_expert logits; s_ex: n_expert doubles of shared
// memory.  On return (after the group's last sync) sh.ids[0..k) hold the ids and sh.val[0..k) the renormalised weights.
template<int PER, class Sync>
__device__ __forceinline__ void route_softmax(const float* __restrict__ l, int n_expert, int k, int tid, int nt,
                                              double* s_ex, RouterShared& sh) {
    float lv[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = j * nt + tid;
        lv[j] = e < n_expert ? l[e] : -INFINITY;
        mx = fmaxf(mx, lv[j]);
    }
    mx = warp_max(mx);
    if ((tid & 31) == 0) sh.rv[tid >> 5] = mx;
    Sync::sync();
    mx = sh.rv[0];
    for (int q = 1; q < (nt >> 5); ++q) mx = fmaxf(mx, sh.rv[q]);
    Sync::sync();

    double ex[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = j * nt + tid;
        ex[j] = e < n_expert ? exp((double) lv[j] - (double) mx) : 0.0;
        if (e < n_expert) s_ex[e] = ex[j];
    }
    Sync::sync();
    if (tid == 0) {
        double sum = 0.0;
        for (int e = 0; e < n_expert; ++e) sum += s_ex[e];   // one thread, ascending: the reference's bits
        sh.inv = (float) (1.0 / sum);
    }
    Sync::sync();
    const float inv = sh.inv;
    float p[PER], sel[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        p[j] = (j * nt + tid) < n_expert ? (float) (ex[j] * inv) : -INFINITY;
        sel[j] = p[j];
    }
    select_topk<PER, Sync>(sel, p, n_expert, k, tid, nt, sh);
    if (tid == 0) {
        double s = 0.0;
        for (int i = 0; i < k; ++i) s += (double) sh.val[i];
        const double sc = fmax(s, 6.103515625e-05);   // 2^-14
        for (int i = 0; i < k; ++i) sh.val[i] = (float) ((double) sh.val[i] / sc);
    }
    Sync::sync();
}

}  // namespace maya
