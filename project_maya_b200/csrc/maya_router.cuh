// maya_router.cuh - the routers' device code, shared by the stand-alone router kernels and the fused decode layer.
//
// Softmax router, value for value what the reference kernel computes (src/kernels/cuda/router_top10.cu:69-187), so the
// expert ids are bit-exact: float max; exp in double of (double) logit - (double) max; ONE ascending double sum;
// inv = (float) (1 / sum); p = (float) (ex * inv); a stable descending top-k (ties -> lower index); weights
// renormalised in double by max(sum of the k weights, 2^-14).
//
// What differs is only how the result is reached, never its bits:
//   * the sum: 1 / sum is rounded to float, so a tree sum decides it whenever the float results at both ends of the
//     tree sum's error interval agree (all terms are positive: any summation order is within (n + 16) * 2^-52 of any
//     other); only when they disagree - about once in a million tokens - one thread repeats the ascending sum;
//   * the selection: with one expert per thread, every thread counts the experts that beat it (keys = value bits over
//     inverted index, unique, so the ranks are a permutation) and ranks 0..k-1 write themselves out: one pass instead of
//     k rounds of arg-max; with more experts per thread p lives in registers, each warp keeps its running arg-max and the
//     k rounds cost one shuffle tree plus one shared-memory exchange each;
//   * the renormalisation: one thread per selected expert divides.
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
    double rd[kRouterMaxWarps];
    alignas(16) unsigned long long cand[kRouterMaxWarps * 8];   // select_rank: every warp's k best keys (k <= 8)
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

// Selection by rank for one expert per thread (nt >= n_expert).  `keys`: n_expert 64-bit words of shared memory.  p >= 0
// (or NaN): its bit pattern orders like the value; the low word makes equal values rank by ascending index, the stable
// descending order.  The keys are distinct whatever p holds, so exactly one thread has each rank.
template<class Sync>
__device__ __forceinline__ void select_rank(float p, int n_expert, int k, int tid, unsigned long long* keys,
                                            RouterShared& sh) {
    const unsigned long long mine = ((unsigned long long) __float_as_uint(p) << 32) | (unsigned) (0xffffffffu - (unsigned) tid);
    if (tid < n_expert) keys[tid] = mine;
    if (k <= 8) {
        // Two levels: a key's rank among its own warp's 32 keys first; the k best of every warp are the only candidates
        // for the global k best (whatever beats a global winner is itself a global winner, hence among its warp's k
        // best), and a candidate's rank among the candidates is its global rank whenever that is below k.  16 + 32
        // shared-memory reads a thread instead of 128; the ids and their order are the same.
        for (int i = tid; i < kRouterMaxWarps * 8; i += 32) sh.cand[i] = 0ull;   // (every warp writes all: no assumption on the
                                                                                 // group's size) a key is never 0: its low word is not
        Sync::sync();
        int lr = 0;
        if (tid < n_expert) {
            const int w0 = tid & ~31;
            if (w0 + 32 <= n_expert) {                        // the whole warp's keys exist: eight reads in flight at a time
                const ulonglong2* k2 = (const ulonglong2*) (keys + w0);
#pragma unroll
                for (int j0 = 0; j0 < 16; j0 += 8) {
                    ulonglong2 o[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) o[j] = k2[j0 + j];
#pragma unroll
                    for (int j = 0; j < 8; ++j) lr += (o[j].x > mine) + (o[j].y > mine);
                }
            } else {
                for (int a = w0; a < n_expert; ++a) lr += keys[a] > mine;
            }
            if (lr < k) sh.cand[(tid >> 5) * 8 + lr] = mine;
        }
        Sync::sync();
        if (tid < n_expert && lr < k) {
            int rank = 0;
            const ulonglong2* c2 = (const ulonglong2*) sh.cand;
#pragma unroll
            for (int j0 = 0; j0 < kRouterMaxWarps * 4; j0 += 8) {
                ulonglong2 o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = c2[j0 + j];
#pragma unroll
                for (int j = 0; j < 8; ++j) rank += (o[j].x > mine) + (o[j].y > mine);
            }
            if (rank < k) { sh.ids[rank] = tid; sh.val[rank] = p; }
        }
        Sync::sync();
        return;
    }
    Sync::sync();
    if (tid < n_expert) {
        int rank = 0;
        const int n2 = n_expert & ~1;
        const ulonglong2* k2 = (const ulonglong2*) keys;
#pragma unroll 8
        for (int j = 0; j < n2 / 2; ++j) {
            const ulonglong2 o = k2[j];
            rank += (o.x > mine) + (o.y > mine);
        }
        if (n2 < n_expert) rank += keys[n2] > mine;
        if (rank < k) { sh.ids[rank] = tid; sh.val[rank] = p; }
    }
    Sync::sync();
}

// One token's softmax routing by the calling thread group.  l: n_expert logits; s_ex: n_expert doubles of shared
// memory, 16-byte aligned.  On return (after the group's last sync) sh.ids[0..k) hold the ids and sh.val[0..k) the
// renormalised weights.
template<int PER, class Sync>
__device__ __forceinline__ void route_softmax(const float* __restrict__ l, int n_expert, int k, int tid, int nt,
                                              double* s_ex, RouterShared& sh) {
    const int nw = nt >> 5;
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
    for (int q = 1; q < nw; ++q) mx = fmaxf(mx, sh.rv[q]);

    double ex[PER], part = 0.0;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = j * nt + tid;
        ex[j] = e < n_expert ? exp((double) lv[j] - (double) mx) : 0.0;
        if (e < n_expert) s_ex[e] = ex[j];
        part += ex[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if ((tid & 31) == 0) sh.rd[tid >> 5] = part;
    Sync::sync();
    double tree = sh.rd[0];
    for (int q = 1; q < nw; ++q) tree += sh.rd[q];
    // every thread holds the same tree sum; the ascending sum lies within tol of it
    const double tol = (double) (n_expert + 16) * 2.220446049250313e-16;
    float inv = (float) (1.0 / (tree * (1.0 - tol)));
    if (inv != (float) (1.0 / (tree * (1.0 + tol)))) {     // group-uniform
        if (tid == 0) {
            double sum = 0.0;
            for (int e = 0; e < n_expert; ++e) sum += s_ex[e];   // one thread, ascending: the reference's bits
            sh.inv = (float) (1.0 / sum);
        }
        Sync::sync();
        inv = sh.inv;
        Sync::sync();                                            // s_ex is reused below
    }
    float p[PER], sel[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        p[j] = (j * nt + tid) < n_expert ? (float) (ex[j] * inv) : -INFINITY;
        sel[j] = p[j];
    }
    if constexpr (PER == 1) select_rank<Sync>(p[0], n_expert, k, tid, (unsigned long long*) s_ex, sh);
    else select_topk<PER, Sync>(sel, p, n_expert, k, tid, nt, sh);
    // weights renormalised in double by max(their sum in selection order, 2^-14): every thread adds, k threads divide
    double s = 0.0;
    for (int i = 0; i < k; ++i) s += (double) sh.val[i];
    const double sc = fmax(s, 6.103515625e-05);   // 2^-14
    const float mine = tid < k ? (float) ((double) sh.val[tid] / sc) : 0.0f;
    Sync::sync();
    if (tid < k) sh.val[tid] = mine;
    Sync::sync();
}

// One token's sigmoid routing (router_sigmoid.cu:29-74, glm_batch.cu:2063-2100): p = sigmoid(logit) in FP32, selection on
// p + bias (bias NULL: none), the stable descending top-k, weights from the unbiased p - divided in double by
// max(their sum, 2^-14) when norm_w - times w_scale.  On return sh.ids[0..k) / sh.val[0..k) hold ids and final weights.
template<int PER, class Sync>
__device__ __forceinline__ void route_sigmoid(const float* __restrict__ l, const float* __restrict__ bias, int n_expert, int k,
                                              float w_scale, int norm_w, int tid, int nt, RouterShared& sh) {
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
    select_topk<PER, Sync>(sel, p, n_expert, k, tid, nt, sh);
    if (tid == 0) {
        double s = 0.0;
        for (int i = 0; i < k; ++i) s += (double) sh.val[i];
        const double sc = fmax(s, 6.103515625e-05);
        for (int i = 0; i < k; ++i) {
            float w = sh.val[i];
            if (norm_w) w = (float) ((double) w / sc);
            sh.val[i] = w * w_scale;
        }
    }
    Sync::sync();
}

}  // namespace maya
