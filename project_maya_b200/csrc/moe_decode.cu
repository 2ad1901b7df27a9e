// moe_decode.cu - the decode-side routed experts: gate/up + SwiGLU + q8_1(h), down + weighted combine, the
// window form that reads each distinct expert once for several tokens, and the grouped "native" form.
//
// Reference entry points replaced: glmf::moe_gate_up / moe_down (src/kernels/cuda/glm_fast.cu:4797-5006, launchers
// :7265-7310, :7387-7417), glmf::moe_win_experts (:7545-7736), native_expert_grouped (src/kernels/cuda/iq_kernels.cu:
// 1077-1194), native_moe_combine (src/kernels/cuda/native_moe.cu:34-85).
//
// All forms run on the same two kernels over GROUPS: a group is one expert blob plus the entries (token column,
// destination slot) that use it.  A plan of k experts for one token is k groups of one entry; a window is the
// distinct experts of T tokens; the native form passes its groups directly.  Weights are decoded once per group and
// dotted with every entry's activation column, and every (row, entry) sum is accumulated in one fixed order, so an
// entry's result does not depend on which other entries share its group.
#include <math.h>

#include <cstdio>
#include <mutex>

#include "maya_dots.cuh"
#include "maya_internal.cuh"
#include "maya_peer_ar.cuh"
#include "maya_stream.cuh"

namespace maya {
namespace {

constexpr int kGuRows = 32;     // h values per block: one q8_1 block of h
constexpr int kGuWarps = 16;    // each warp: 2 gate + 2 up rows
constexpr int kDownWarps = 8;
constexpr int kDownRowsPerWarp = 4;
constexpr int kDownRows = kDownWarps * kDownRowsPerWarp;
constexpr int kNC = 4;          // activation columns dotted per decode pass

// How a kernel finds its groups.
struct Groups {
    const unsigned long long* ptr;   // [n] blob addresses (0 = skipped)
    const int* start;                // [n + 1] entry ranges, or NULL: group g has the single entry g
    const int* n_groups;             // device count, or NULL: the launch's grid says
    const int* ent_slot;             // [entries] the entry's h / partial slot, or NULL: the entry index
    const int* ent_tok;              // [entries] the entry's activation column, or NULL: slot >> 3 (tok_from_slot) or 0
    const int* ent_out;              // [entries] the entry's output row (down), or NULL: its slot
    const int* skip;                 // optional "do nothing" flag
    int tok_from_slot;
    int cap_entries;                 // > 0: entry numbers at or beyond it are not touched (the scratch ends there)
    __device__ __forceinline__ int slot(int e) const { return ent_slot ? ent_slot[e] : e; }
    __device__ __forceinline__ int tok(int e) const { return ent_tok ? ent_tok[e] : (tok_from_slot ? slot(e) >> 3 : 0); }
    __device__ __forceinline__ int out_row(int e) const { return ent_out ? ent_out[e] : slot(e); }
};

// ------------------------------------------------------------------------------------------------ gate / up
// grid (n_ff / 32, groups [+ 1 shared-down row of blocks]); block 512.
template<int T>
__global__ void __launch_bounds__(kGuWarps * 32, 2) gate_up_kernel(Groups G, int n_groups_grid, int n_embd, int n_ff,
                                                                size_t up_off, float limit,
                                                                const uint8_t* __restrict__ xq, size_t xq_stride,
                                                                uint8_t* __restrict__ hq,
                                                                // the shared expert's down rows (blockIdx.y == groups)
                                                                const uint8_t* __restrict__ sh_down, int sh_type,
                                                                const uint8_t* __restrict__ sh_hq, int n_ff_sh,
                                                                float* __restrict__ sh_out);

template<int TS>
__device__ __forceinline__ void shared_down_rows(const uint8_t* sh_down, const uint8_t* sh_hq, int n_ff_sh, int n_embd,
                                                 int chunk, int n_chunks, float* sh_out, uint8_t* smem) {
    uint32_t* s_tab = (uint32_t*) smem;
    int4* q; float* d; int* is;
    const int nblk = n_ff_sh / 32;
    const XCols x = xcols_carve(smem + Fmt<TS>::tab_words * 4, nblk, 1, &q, &d, &is);
    load_tab<TS>(s_tab);
    xcols_stage_p<Dec<TS>::xblk>(sh_hq, 0, nblk, 1, q, d, is);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int per = (n_embd + n_chunks - 1) / n_chunks;
    const int r1 = min(n_embd, (chunk + 1) * per);
    const size_t rb = row_bytes(TS, n_ff_sh);
    for (int r = chunk * per + 2 * warp; r < r1; r += 2 * nw) {
        const uint8_t* rows[2] = {sh_down + (size_t) r * rb, sh_down + (size_t) min(r + 1, r1 - 1) * rb};
        float o[2][1];
        rows_dot<TS, 2, 1>(rows, x, 1, n_ff_sh, lane, s_tab, o);
        if (lane == 0) {
            sh_out[r] = o[0][0];
            if (r + 1 < r1) sh_out[r + 1] = o[1][0];
        }
    }
}

template<int T>
__global__ void __launch_bounds__(kGuWarps * 32, 2) gate_up_kernel(Groups G, int n_groups_grid, int n_embd, int n_ff,
                                                                size_t up_off, float limit,
                                                                const uint8_t* __restrict__ xq, size_t xq_stride,
                                                                uint8_t* __restrict__ hq,
                                                                const uint8_t* __restrict__ sh_down, int sh_type,
                                                                const uint8_t* __restrict__ sh_hq, int n_ff_sh,
                                                                float* __restrict__ sh_out) {
    extern __shared__ __align__(16) uint8_t s_raw[];
    if (G.skip != nullptr && *G.skip) return;
    const int g = blockIdx.y, chunk = blockIdx.x;
    if (g == n_groups_grid) {   // the extra row of blocks: the shared expert's down projection, spread over the chunks
        switch (sh_type) {
            case MAYA_Q8_0: shared_down_rows<MAYA_Q8_0>(sh_down, sh_hq, n_ff_sh, n_embd, chunk, gridDim.x, sh_out, s_raw); break;
            case MAYA_Q4_K: shared_down_rows<MAYA_Q4_K>(sh_down, sh_hq, n_ff_sh, n_embd, chunk, gridDim.x, sh_out, s_raw); break;
            case MAYA_IQ2_S: shared_down_rows<MAYA_IQ2_S>(sh_down, sh_hq, n_ff_sh, n_embd, chunk, gridDim.x, sh_out, s_raw); break;
            default: shared_down_rows<MAYA_IQ3_S>(sh_down, sh_hq, n_ff_sh, n_embd, chunk, gridDim.x, sh_out, s_raw); break;
        }
        return;
    }
    if (G.n_groups != nullptr && g >= *G.n_groups) return;
    const unsigned long long ptr = G.ptr[g];
    if (ptr == 0ull) return;
    const int e0 = G.start ? G.start[g] : g;
    int e1 = G.start ? G.start[g + 1] : g + 1;
    if (G.cap_entries > 0) e1 = min(e1, G.cap_entries);      // an inconsistent start table must not reach past the scratch
    if (e1 <= e0 || e0 < 0) return;

    __shared__ float s_g[kNC][kGuRows], s_u[kNC][kGuRows];
    uint32_t* s_tab = (uint32_t*) s_raw;
    int4* q; float* d; int* is;
    const int nblk = n_embd / 32;
    const XCols x = xcols_carve(s_raw + Fmt<T>::tab_words * 4, nblk, kNC, &q, &d, &is);
    load_tab<T>(s_tab);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t rb = row_bytes(T, n_embd);
    const uint8_t* blob = (const uint8_t*) ptr;
    constexpr int RPW = kGuRows / kGuWarps;   // 2
    const uint8_t* rows[2 * RPW];
#pragma unroll
    for (int j = 0; j < RPW; ++j) {
        const int r = chunk * kGuRows + warp * RPW + j;
        rows[j] = blob + (size_t) r * rb;
        rows[RPW + j] = blob + up_off + (size_t) r * rb;
    }
    // The warp's rows are asked into L2 now, while the block stages its columns: the dots' own loads (one dependent
    // round per 32 calls of a row) then wait for L2 instead of device memory from the second round on.
    if (lane == 0) {
        bulk_prefetch_l2(rows[0], (uint32_t) (RPW * rb));
        bulk_prefetch_l2(rows[RPW], (uint32_t) (RPW * rb));
    }
    for (int eb = e0; eb < e1; eb += kNC) {
        const int nc = min(kNC, e1 - eb);
        __syncthreads();   // the previous pass is done with the staged columns and s_g / s_u
        for (int c = 0; c < nc; ++c) {
            const int tok = G.tok(eb + c);
            xcols_stage_p<Dec<T>::xblk, T == MAYA_IQ1_S>(xq + (size_t) tok * xq_stride, 0, nblk, 1, q + (size_t) 2 * c * nblk, d + (size_t) c * nblk,
                        is + (size_t) c * nblk);
        }
        __syncthreads();
        float o[2 * RPW][kNC];
        if (nc == 1) {
            float o1[2 * RPW][1];
            rows_dot<T, 2 * RPW, 1>(rows, x, 1, n_embd, lane, s_tab, o1);
#pragma unroll
            for (int j = 0; j < 2 * RPW; ++j) o[j][0] = o1[j][0];
        } else {
            rows_dot<T, 2 * RPW, kNC>(rows, x, nc, n_embd, lane, s_tab, o);
        }
        if (lane == 0) {
#pragma unroll
            for (int j = 0; j < RPW; ++j)
#pragma unroll
                for (int c = 0; c < kNC; ++c)
                    if (c < nc) { s_g[c][warp * RPW + j] = o[j][c]; s_u[c][warp * RPW + j] = o[RPW + j][c]; }
        }
        __syncthreads();
        if (warp < nc) {
            const int dst = G.slot(eb + warp);
            q8_1_store_warp(swiglu(s_g[warp][lane], s_u[warp][lane], limit),
                            hq + ((size_t) dst * (n_ff / 32) + chunk) * kQ81Bytes, lane);
        }
    }
}

// A layer whose up rows have their own type (NativeExpertLayout::u_type, iq_kernels.hpp:73-77; the native grouped path
// only): the gate rows and the up rows of a warp are dotted by two calls of their own decoder.  A row's result does not
// depend on which rows share a call, so with TG == TU this is gate_up_kernel's arithmetic bit for bit.
template<int TG, int TU>
__global__ void __launch_bounds__(kGuWarps * 32) gate_up_mixed_kernel(Groups G, int n_embd, int n_ff, size_t up_off, float limit,
                                                                      const uint8_t* __restrict__ xq, size_t xq_stride,
                                                                      uint8_t* __restrict__ hq) {
    extern __shared__ __align__(16) uint8_t s_raw[];
    if (G.skip != nullptr && *G.skip) return;
    const int g = blockIdx.y, chunk = blockIdx.x;
    if (G.n_groups != nullptr && g >= *G.n_groups) return;
    const unsigned long long ptr = G.ptr[g];
    if (ptr == 0ull) return;
    const int e0 = G.start ? G.start[g] : g;
    int e1 = G.start ? G.start[g + 1] : g + 1;
    if (G.cap_entries > 0) e1 = min(e1, G.cap_entries);
    if (e1 <= e0 || e0 < 0) return;

    __shared__ float s_g[kNC][kGuRows], s_u[kNC][kGuRows];
    uint32_t* s_tab_g = (uint32_t*) s_raw;
    uint32_t* s_tab_u = s_tab_g + Fmt<TG>::tab_words;
    int4* q; float* d; int* is;
    const int nblk = n_embd / 32;
    const XCols x = xcols_carve((uint8_t*) (s_tab_u + Fmt<TU>::tab_words), nblk, kNC, &q, &d, &is);
    load_tab<TG>(s_tab_g);
    load_tab<TU>(s_tab_u);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t rbg = row_bytes(TG, n_embd), rbu = row_bytes(TU, n_embd);
    const uint8_t* blob = (const uint8_t*) ptr;
    constexpr int RPW = kGuRows / kGuWarps;   // 2
    const uint8_t* grow[RPW];
    const uint8_t* urow[RPW];
#pragma unroll
    for (int j = 0; j < RPW; ++j) {
        const int r = chunk * kGuRows + warp * RPW + j;
        grow[j] = blob + (size_t) r * rbg;
        urow[j] = blob + up_off + (size_t) r * rbu;
    }
    for (int eb = e0; eb < e1; eb += kNC) {
        const int nc = min(kNC, e1 - eb);
        __syncthreads();
        // the two types read the same staged columns: the planar form of the wider call span serves both
        constexpr int XL = Dec<TG>::xblk > Dec<TU>::xblk ? Dec<TG>::xblk : Dec<TU>::xblk;
        for (int c = 0; c < nc; ++c)
            xcols_stage_p<XL>(xq + (size_t) G.tok(eb + c) * xq_stride, 0, nblk, 1, q + (size_t) 2 * c * nblk, d + (size_t) c * nblk,
                              is + (size_t) c * nblk);
        __syncthreads();
        float og[RPW][kNC], ou[RPW][kNC];
        if (nc == 1) {
            float a[RPW][1], b[RPW][1];
            rows_dot<TG, RPW, 1, XL>(grow, x, 1, n_embd, lane, s_tab_g, a);
            rows_dot<TU, RPW, 1, XL>(urow, x, 1, n_embd, lane, s_tab_u, b);
#pragma unroll
            for (int j = 0; j < RPW; ++j) { og[j][0] = a[j][0]; ou[j][0] = b[j][0]; }
        } else {
            rows_dot<TG, RPW, kNC, XL>(grow, x, nc, n_embd, lane, s_tab_g, og);
            rows_dot<TU, RPW, kNC, XL>(urow, x, nc, n_embd, lane, s_tab_u, ou);
        }
        if (lane == 0) {
#pragma unroll
            for (int j = 0; j < RPW; ++j)
#pragma unroll
                for (int c = 0; c < kNC; ++c)
                    if (c < nc) { s_g[c][warp * RPW + j] = og[j][c]; s_u[c][warp * RPW + j] = ou[j][c]; }
        }
        __syncthreads();
        if (warp < nc) {
            const int dst = G.slot(eb + warp);
            q8_1_store_warp(swiglu(s_g[warp][lane], s_u[warp][lane], limit),
                            hq + ((size_t) dst * (n_ff / 32) + chunk) * kQ81Bytes, lane);
        }
    }
}

// ------------------------------------------------------------------------------------------------ down, plan form
// One token: block = kDownRows output rows; warp w computes 4 of them for every plan entry in turn, then combines in
// plan order: m = 0; m = fma(w_i, part_i, m); out = m [+ cpu_part] + sh_out (the reference's chain, glm_fast.cu:4999-5005).
template<int T>
__global__ void __launch_bounds__(kDownWarps * 32) down_plan_kernel(maya_moe_plan P, int k, int n_embd, int n_ff,
                                                                    size_t down_off, const uint8_t* __restrict__ hq,
                                                                    const float* __restrict__ sh_out,
                                                                    float* __restrict__ out) {
    extern __shared__ __align__(16) uint8_t s_raw[];
    if (P.skip != nullptr && *P.skip) return;
    uint32_t* s_tab = (uint32_t*) s_raw;
    int4* q; float* d; int* is;
    const int nblk = n_ff / 32;
    const XCols x = xcols_carve(s_raw + Fmt<T>::tab_words * 4, nblk, k, &q, &d, &is);
    load_tab<T>(s_tab);
    xcols_stage_p<Dec<T>::xblk, T == MAYA_IQ1_S>(hq, (size_t) nblk * kQ81Bytes, nblk, k, q, d, is);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r0 = (int) blockIdx.x * kDownRows + warp * kDownRowsPerWarp;
    if (r0 >= n_embd) return;
    const size_t rb = row_bytes(T, n_ff);
    float m[kDownRowsPerWarp];
#pragma unroll
    for (int j = 0; j < kDownRowsPerWarp; ++j) m[j] = 0.0f;
    for (int i = 0; i < k; ++i) {
        const unsigned long long ptr = P.plan_ptr[i];
        const float wi = P.plan_w[i];
        float o[kDownRowsPerWarp][1];
        if (ptr != 0ull) {
            const uint8_t* rows[kDownRowsPerWarp];
#pragma unroll
            for (int j = 0; j < kDownRowsPerWarp; ++j)
                rows[j] = (const uint8_t*) ptr + down_off + (size_t) min(r0 + j, n_embd - 1) * rb;
            XCols xi = x;
            xi.q += (size_t) 2 * i * nblk; xi.d += (size_t) i * nblk; xi.isum += (size_t) i * nblk;
            rows_dot<T, kDownRowsPerWarp, 1>(rows, xi, 1, n_ff, lane, s_tab, o);
        } else {
#pragma unroll
            for (int j = 0; j < kDownRowsPerWarp; ++j) o[j][0] = 0.0f;
        }
#pragma unroll
        for (int j = 0; j < kDownRowsPerWarp; ++j) m[j] = __fmaf_rn(wi, o[j][0], m[j]);
    }
    if (lane < kDownRowsPerWarp && r0 + lane < n_embd) {
        float v = 0.0f;
#pragma unroll
        for (int j = 0; j < kDownRowsPerWarp; ++j) if (lane == j) v = m[j];
        const int r = r0 + lane;
        if (P.cpu_flag != nullptr && *P.cpu_flag) v = __fadd_rn(v, P.cpu_part[r]);
        out[r] = __fadd_rn(v, sh_out != nullptr ? sh_out[r] : 0.0f);
    }
}

// ------------------------------------------------------------------------------------------------ down, group form
// grid (n_embd / kDownRows, groups): part[dst][row] = down[row] . hq[dst] for every entry of the group (unweighted).
template<int T>
__global__ void __launch_bounds__(kDownWarps * 32, 4) down_groups_kernel(Groups G, int n_embd, int n_ff, size_t down_off,
                                                                      const uint8_t* __restrict__ hq,
                                                                      float* __restrict__ part) {
    extern __shared__ __align__(16) uint8_t s_raw[];
    if (G.skip != nullptr && *G.skip) return;
    const int g = blockIdx.y;
    if (G.n_groups != nullptr && g >= *G.n_groups) return;
    const unsigned long long ptr = G.ptr[g];
    if (ptr == 0ull) return;
    const int e0 = G.start ? G.start[g] : g;
    int e1 = G.start ? G.start[g + 1] : g + 1;
    if (G.cap_entries > 0) e1 = min(e1, G.cap_entries);      // an inconsistent start table must not reach past the scratch
    if (e1 <= e0 || e0 < 0) return;
    uint32_t* s_tab = (uint32_t*) s_raw;
    int4* q; float* d; int* is;
    const int nblk = n_ff / 32;
    const XCols x = xcols_carve(s_raw + Fmt<T>::tab_words * 4, nblk, kNC, &q, &d, &is);
    load_tab<T>(s_tab);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r0 = (int) blockIdx.x * kDownRows + warp * kDownRowsPerWarp;
    const size_t rb = row_bytes(T, n_ff);
    const uint8_t* rows[kDownRowsPerWarp];
#pragma unroll
    for (int j = 0; j < kDownRowsPerWarp; ++j)
        rows[j] = (const uint8_t*) ptr + down_off + (size_t) min(r0 + j, n_embd - 1) * rb;
    if (lane == 0 && r0 + kDownRowsPerWarp <= n_embd)             // the warp's rows into L2 while the columns are staged
        bulk_prefetch_l2(rows[0], (uint32_t) (kDownRowsPerWarp * rb));
    for (int eb = e0; eb < e1; eb += kNC) {
        const int nc = min(kNC, e1 - eb);
        __syncthreads();
        for (int c = 0; c < nc; ++c) {
            const int dst = G.slot(eb + c);
            xcols_stage_p<Dec<T>::xblk, T == MAYA_IQ1_S>(hq + (size_t) dst * nblk * kQ81Bytes, 0, nblk, 1, q + (size_t) 2 * c * nblk, d + (size_t) c * nblk,
                        is + (size_t) c * nblk);
        }
        __syncthreads();
        if (r0 >= n_embd) continue;
        float o[kDownRowsPerWarp][kNC];
        if (nc == 1) {
            float o1[kDownRowsPerWarp][1];
            rows_dot<T, kDownRowsPerWarp, 1>(rows, x, 1, n_ff, lane, s_tab, o1);
#pragma unroll
            for (int j = 0; j < kDownRowsPerWarp; ++j) o[j][0] = o1[j][0];
        } else {
            rows_dot<T, kDownRowsPerWarp, kNC>(rows, x, nc, n_ff, lane, s_tab, o);
        }
        if (lane == 0) {
#pragma unroll
            for (int c = 0; c < kNC; ++c) {
                if (c >= nc) continue;
                const int dst = G.out_row(eb + c);
#pragma unroll
                for (int j = 0; j < kDownRowsPerWarp; ++j)
                    if (r0 + j < n_embd) part[(size_t) dst * n_embd + r0 + j] = o[j][c];
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ window grouping
// Entries i = t * 8 + j (token t, plan slot j) with a non-zero blob address are grouped by address: groups in order of
// first appearance, members in ascending i.  One block; T * 8 <= 128 entries.
__global__ void __launch_bounds__(128) win_group_kernel(const unsigned long long* __restrict__ plan_ptr, int T, int k,
                                                        unsigned long long* __restrict__ grp_ptr,
                                                        int* __restrict__ grp_start, int* __restrict__ grp_ent,
                                                        int* __restrict__ n_groups) {
    __shared__ unsigned long long s_ptr[128];
    __shared__ int s_leader[128], s_gidx[128], s_cnt[129];
    const int i = threadIdx.x, n = T * 8;
    const int t = i >> 3, j = i & 7;
    s_ptr[i] = (i < n && j < k) ? plan_ptr[i] : 0ull;
    __syncthreads();
    const unsigned long long p = s_ptr[i];
    int leader = -1;
    if (p != 0ull) {
        leader = i;
        for (int f = 0; f < i; ++f)
            if (s_ptr[f] == p) { leader = f; break; }
    }
    s_leader[i] = leader;
    __syncthreads();
    // group index of a leader = leaders before it
    int gi = 0;
    if (leader == i)
        for (int f = 0; f < i; ++f) gi += (s_leader[f] == f);
    s_gidx[i] = gi;
    s_cnt[i] = 0;
    if (i == 0) s_cnt[128] = 0;
    __syncthreads();
    const int my_group = leader >= 0 ? s_gidx[leader] : -1;
    int rank = 0;   // members of my group before me
    if (leader >= 0)
        for (int f = 0; f < i; ++f) rank += (s_leader[f] == leader);
    if (leader >= 0) atomicAdd(&s_cnt[my_group], 1);
    __syncthreads();
    // exclusive scan of the counts by every thread for its own group (<= 128 groups)
    int ng = 0;
    for (int f = 0; f < 128; ++f) ng += (s_leader[f] == f);
    int start = 0;
    if (leader >= 0)
        for (int f = 0; f < my_group; ++f) start += s_cnt[f];
    if (leader >= 0) grp_ent[start + rank] = i;
    if (leader == i) { grp_ptr[my_group] = p; grp_start[my_group] = start; }
    if (i == 0) {
        int total = 0;
        for (int f = 0; f < ng; ++f) total += s_cnt[f];
        grp_start[ng] = total;
        *n_groups = ng;
    }
    (void) t;
}

// out[t][r] = fma chain over the token's plan slots in plan order (a skipped slot contributes w * 0, as the plan
// kernel's zero partial does) [+ cpu_part] + sh_out: down_plan_kernel's tail, value for value.
__global__ void __launch_bounds__(256) win_combine_kernel(const unsigned long long* __restrict__ plan_ptr,
                                                          const float* __restrict__ plan_w, int k, int n_embd,
                                                          const float* __restrict__ part,
                                                          const float* __restrict__ cpu_part,
                                                          const int* __restrict__ cpu_flag,
                                                          const float* __restrict__ sh_out, float* __restrict__ out,
                                                          size_t out_stride) {
    const int t = blockIdx.y, r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_embd) return;
    float m = 0.0f;
    for (int j = 0; j < k; ++j) {
        const float pv = plan_ptr[t * 8 + j] != 0ull ? part[((size_t) t * 8 + j) * n_embd + r] : 0.0f;
        m = __fmaf_rn(plan_w[t * 8 + j], pv, m);
    }
    if (cpu_flag != nullptr && cpu_flag[t]) m = __fadd_rn(m, cpu_part[(size_t) t * n_embd + r]);
    out[(size_t) t * out_stride + r] = __fadd_rn(m, sh_out != nullptr ? sh_out[(size_t) t * n_embd + r] : 0.0f);
}

// win_combine_kernel and the cross-rank sum in one launch (the reference follows win_experts with a separate allreduce
// over out[T * n_embd], src/ds4/ds4_model.cu:22822-22828): block b combines its share [q0, q1) (float4 units of the
// contiguous [T][n_embd] output), then runs the rows + flags exchange on it (peer_allreduce_block).
__global__ void __launch_bounds__(256) win_combine_ar_kernel(const unsigned long long* __restrict__ plan_ptr,
                                                             const float* __restrict__ plan_w, int k, int n_embd,
                                                             const float* __restrict__ part,
                                                             const float* __restrict__ cpu_part,
                                                             const int* __restrict__ cpu_flag,
                                                             const float* __restrict__ sh_out, float* out, int n4,
                                                             maya_peer_ar a, int mi, unsigned seq) {
    const int nb = gridDim.x, b = blockIdx.x;
    const int base = n4 / nb, rem = n4 % nb;
    const int q0 = b * base + min(b, rem), q1 = q0 + base + (b < rem ? 1 : 0);
    for (int q = q0 + threadIdx.x; q < q1; q += blockDim.x) {
        const int t = (int) (((size_t) q * 4) / n_embd), r = (int) ((size_t) q * 4 - (size_t) t * n_embd);
        float4 m = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int j = 0; j < k; ++j) {
            float4 pv = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (plan_ptr[t * 8 + j] != 0ull) pv = *(const float4*) (part + ((size_t) t * 8 + j) * n_embd + r);
            const float wj = plan_w[t * 8 + j];
            m.x = __fmaf_rn(wj, pv.x, m.x); m.y = __fmaf_rn(wj, pv.y, m.y); m.z = __fmaf_rn(wj, pv.z, m.z); m.w = __fmaf_rn(wj, pv.w, m.w);
        }
        if (cpu_flag != nullptr && cpu_flag[t]) {
            const float4 c = *(const float4*) (cpu_part + (size_t) t * n_embd + r);
            m.x = __fadd_rn(m.x, c.x); m.y = __fadd_rn(m.y, c.y); m.z = __fadd_rn(m.z, c.z); m.w = __fadd_rn(m.w, c.w);
        }
        float4 s4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (sh_out != nullptr) s4 = *(const float4*) (sh_out + (size_t) t * n_embd + r);
        m.x = __fadd_rn(m.x, s4.x); m.y = __fadd_rn(m.y, s4.y); m.z = __fadd_rn(m.z, s4.z); m.w = __fadd_rn(m.w, s4.w);
        ((float4*) out)[q] = m;
    }
    __syncthreads();
    const unsigned sq = ar_seq_begin(a, seq);
    peer_allreduce_block(out, q0, q1, a, mi, sq, b);
    ar_seq_end(a, seq, sq);
}

// native_moe combine: s = parts[0] * w[0]; s = fma(parts[i], w[i], s); + shared (native_moe.cu:42-47).
__global__ void __launch_bounds__(256) combine_kernel(const float* __restrict__ parts, const float* __restrict__ w,
                                                      const float* __restrict__ shared, float* __restrict__ y,
                                                      int64_t n_embd, int k) {
    const int t = blockIdx.y;
    const int64_t r = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_embd) return;
    const float* p = parts + (size_t) t * k * n_embd;
    const float* wt = w + (size_t) t * k;
    float s = __fmul_rn(p[r], wt[0]);
    for (int i = 1; i < k; ++i) s = __fmaf_rn(p[(size_t) i * n_embd + r], wt[i], s);
    y[(size_t) t * n_embd + r] = shared != nullptr ? __fadd_rn(s, shared[(size_t) t * n_embd + r]) : s;
}

// ------------------------------------------------------------------------------------------------ launch helpers
template<int T>
int launch_gate_up(const Groups& G, int n_groups_grid, int n_embd, int n_ff, size_t up_off, float limit, const void* xq,
                   size_t xq_stride, void* hq, const void* sh_down, int sh_type, const void* sh_hq, int n_ff_sh,
                   float* sh_out, cudaStream_t s) {
    size_t smem = (size_t) Fmt<T>::tab_words * 4 + xcols_bytes(n_embd / 32, kNC);
    if (sh_down != nullptr) {
        const size_t sh = 8192 + xcols_bytes(n_ff_sh / 32, 1);
        if (sh > smem) smem = sh;
    }
    if (smem > 200 * 1024) return refuse(MAYA_ERR_LIMIT);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(gate_up_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess)
        return note_launch("gate_up smem attribute");
    const dim3 grid((unsigned) (n_ff / kGuRows), (unsigned) (n_groups_grid + (sh_down != nullptr ? 1 : 0)));
    gate_up_kernel<T><<<grid, kGuWarps * 32, smem, s>>>(G, n_groups_grid, n_embd, n_ff, up_off, limit, (const uint8_t*) xq,
                                                        xq_stride, (uint8_t*) hq, (const uint8_t*) sh_down, sh_type,
                                                        (const uint8_t*) sh_hq, n_ff_sh, sh_out);
    return note_launch("moe_gate_up");
}

template<int T>
int launch_down_plan(const maya_moe_plan& P, int k, int n_embd, int n_ff, size_t down_off, const void* hq,
                     const float* sh_out, float* out, cudaStream_t s) {
    const size_t smem = (size_t) Fmt<T>::tab_words * 4 + xcols_bytes(n_ff / 32, k);
    if (smem > 200 * 1024) return refuse(MAYA_ERR_LIMIT);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(down_plan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess)
        return note_launch("down smem attribute");
    down_plan_kernel<T><<<(n_embd + kDownRows - 1) / kDownRows, kDownWarps * 32, smem, s>>>(
        P, k, n_embd, n_ff, down_off, (const uint8_t*) hq, sh_out, out);
    return note_launch("moe_down");
}

template<int T>
int launch_down_groups(const Groups& G, int n_groups_grid, int n_embd, int n_ff, size_t down_off, const void* hq,
                       float* part, cudaStream_t s) {
    const size_t smem = (size_t) Fmt<T>::tab_words * 4 + xcols_bytes(n_ff / 32, kNC);
    if (smem > 200 * 1024) return refuse(MAYA_ERR_LIMIT);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(down_groups_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess)
        return note_launch("down_groups smem attribute");
    const dim3 grid((unsigned) ((n_embd + kDownRows - 1) / kDownRows), (unsigned) n_groups_grid);
    down_groups_kernel<T><<<grid, kDownWarps * 32, smem, s>>>(G, n_embd, n_ff, down_off, (const uint8_t*) hq, part);
    return note_launch("down_groups");
}

template<int TG, int TU>
int launch_gate_up_mixed(const Groups& G, int n_groups_grid, int n_embd, int n_ff, size_t up_off, float limit, const void* xq,
                         size_t xq_stride, void* hq, cudaStream_t s) {
    const size_t smem = (size_t) (Fmt<TG>::tab_words + Fmt<TU>::tab_words) * 4 + xcols_bytes(n_embd / 32, kNC);
    if (smem > 200 * 1024) return refuse(MAYA_ERR_LIMIT);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(gate_up_mixed_kernel<TG, TU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess)
        return note_launch("gate_up_mixed smem attribute");
    const dim3 grid((unsigned) (n_ff / kGuRows), (unsigned) n_groups_grid);
    gate_up_mixed_kernel<TG, TU><<<grid, kGuWarps * 32, smem, s>>>(G, n_embd, n_ff, up_off, limit, (const uint8_t*) xq, xq_stride,
                                                                  (uint8_t*) hq);
    return note_launch("moe_gate_up_mixed");
}
template<int TG>
int launch_gate_up_mixed_u(int u_type, const Groups& G, int n_groups_grid, int n_embd, int n_ff, size_t up_off, float limit,
                           const void* xq, size_t xq_stride, void* hq, cudaStream_t s) {
    switch (u_type) {
        case MAYA_Q8_0: return launch_gate_up_mixed<TG, MAYA_Q8_0>(G, n_groups_grid, n_embd, n_ff, up_off, limit, xq, xq_stride, hq, s);
        case MAYA_Q4_K: return launch_gate_up_mixed<TG, MAYA_Q4_K>(G, n_groups_grid, n_embd, n_ff, up_off, limit, xq, xq_stride, hq, s);
        case MAYA_IQ2_S: return launch_gate_up_mixed<TG, MAYA_IQ2_S>(G, n_groups_grid, n_embd, n_ff, up_off, limit, xq, xq_stride, hq, s);
        case MAYA_IQ3_S: return launch_gate_up_mixed<TG, MAYA_IQ3_S>(G, n_groups_grid, n_embd, n_ff, up_off, limit, xq, xq_stride, hq, s);
        default: return refuse(MAYA_ERR_TYPE);
    }
}

#define MAYA_TYPE_SWITCH(type, CALL)                      \
    switch (type) {                                       \
        case MAYA_Q8_0: return CALL(MAYA_Q8_0);           \
        case MAYA_Q4_K: return CALL(MAYA_Q4_K);           \
        case MAYA_IQ2_S: return CALL(MAYA_IQ2_S);         \
        case MAYA_IQ3_S: return CALL(MAYA_IQ3_S);         \
        case MAYA_Q5_K: return CALL(MAYA_Q5_K);           \
        case MAYA_Q6_K: return CALL(MAYA_Q6_K);           \
        case MAYA_IQ4_XS: return CALL(MAYA_IQ4_XS);       \
        case MAYA_IQ3_XXS: return CALL(MAYA_IQ3_XXS);     \
        case MAYA_IQ2_XXS: return CALL(MAYA_IQ2_XXS);     \
        case MAYA_IQ1_S: return CALL(MAYA_IQ1_S);         \
        default: return refuse(MAYA_ERR_TYPE);            \
    }

int check_shapes(int gu_type, int d_type, int k, int n_embd, int n_ff) {
    if (gu_type >= 0 && !type_qk(gu_type)) return MAYA_ERR_TYPE;
    if (d_type >= 0 && !type_qk(d_type)) return MAYA_ERR_TYPE;
    if (k < 1 || k > MAYA_MAX_K) return MAYA_ERR_LIMIT;
    if (n_embd <= 0 || n_ff <= 0 || n_ff % 32 || n_embd % 32) return MAYA_ERR_ARG;
    if (gu_type >= 0 && n_embd % type_qk(gu_type)) return MAYA_ERR_ARG;
    if (d_type >= 0 && n_ff % type_qk(d_type)) return MAYA_ERR_ARG;
    return MAYA_OK;
}

}  // namespace

// Used by the whole-layer entry point (moe_layer.cu) and the C entry points below.
int gate_up_groups(int gu_type, const GroupArgs& A, int n_groups_grid, int n_embd, int n_ff, size_t up_off, float limit,
                   const void* xq, size_t xq_stride, void* hq, const void* sh_down, int sh_type, const void* sh_hq,
                   int n_ff_sh, float* sh_out, cudaStream_t s) {
    Groups G{A.ptr, A.start, A.n_groups, A.ent_slot, A.ent_tok, A.ent_out, A.skip, A.tok_from_slot, A.cap_entries};
#define CALL(TT) launch_gate_up<TT>(G, n_groups_grid, n_embd, n_ff, up_off, limit, xq, xq_stride, hq, sh_down, sh_type, sh_hq, n_ff_sh, sh_out, s)
    MAYA_TYPE_SWITCH(gu_type, CALL)
#undef CALL
}

// gate_up_groups for a layer whose up rows are of another type than its gate rows (no shared-expert rows in the launch).
int gate_up_groups_mixed(int g_type, int u_type, const GroupArgs& A, int n_groups_grid, int n_embd, int n_ff, size_t up_off,
                         float limit, const void* xq, size_t xq_stride, void* hq, cudaStream_t s) {
    Groups G{A.ptr, A.start, A.n_groups, A.ent_slot, A.ent_tok, A.ent_out, A.skip, A.tok_from_slot, A.cap_entries};
    switch (g_type) {
        case MAYA_Q8_0: return launch_gate_up_mixed_u<MAYA_Q8_0>(u_type, G, n_groups_grid, n_embd, n_ff, up_off, limit, xq, xq_stride, hq, s);
        case MAYA_Q4_K: return launch_gate_up_mixed_u<MAYA_Q4_K>(u_type, G, n_groups_grid, n_embd, n_ff, up_off, limit, xq, xq_stride, hq, s);
        case MAYA_IQ2_S: return launch_gate_up_mixed_u<MAYA_IQ2_S>(u_type, G, n_groups_grid, n_embd, n_ff, up_off, limit, xq, xq_stride, hq, s);
        case MAYA_IQ3_S: return launch_gate_up_mixed_u<MAYA_IQ3_S>(u_type, G, n_groups_grid, n_embd, n_ff, up_off, limit, xq, xq_stride, hq, s);
        default: return refuse(MAYA_ERR_TYPE);
    }
}
int down_groups(int d_type, const GroupArgs& A, int n_groups_grid, int n_embd, int n_ff, size_t down_off, const void* hq,
                float* part, cudaStream_t s) {
    Groups G{A.ptr, A.start, A.n_groups, A.ent_slot, A.ent_tok, A.ent_out, A.skip, A.tok_from_slot, A.cap_entries};
#define CALL(TT) launch_down_groups<TT>(G, n_groups_grid, n_embd, n_ff, down_off, hq, part, s)
    MAYA_TYPE_SWITCH(d_type, CALL)
#undef CALL
}
int down_plan(int d_type, const maya_moe_plan& P, int k, int n_embd, int n_ff, size_t down_off, const void* hq,
              const float* sh_out, float* out, cudaStream_t s) {
#define CALL(TT) launch_down_plan<TT>(P, k, n_embd, n_ff, down_off, hq, sh_out, out, s)
    MAYA_TYPE_SWITCH(d_type, CALL)
#undef CALL
}
int win_combine(const unsigned long long* plan_ptr, const float* plan_w, int T, int k, int n_embd, const float* part,
                const float* cpu_part, const int* cpu_flag, const float* sh_out, float* out, size_t out_stride,
                cudaStream_t s) {
    const dim3 grid((unsigned) ((n_embd + 255) / 256), (unsigned) T);
    win_combine_kernel<<<grid, 256, 0, s>>>(plan_ptr, plan_w, k, n_embd, part, cpu_part, cpu_flag, sh_out, out, out_stride);
    return note_launch("moe_win_combine");
}

int win_combine_ar(const unsigned long long* plan_ptr, const float* plan_w, int T, int k, int n_embd, const float* part,
                   const float* cpu_part, const int* cpu_flag, const float* sh_out, float* out, const maya_peer_ar& a, int mi,
                   unsigned seq, cudaStream_t s) {
    const int n4 = (int) ((size_t) T * n_embd / 4);
    int blocks = (n4 + 255) / 256;
    if (blocks > MAYA_PEER_AR_BLOCKS) blocks = MAYA_PEER_AR_BLOCKS;
    win_combine_ar_kernel<<<blocks, 256, 0, s>>>(plan_ptr, plan_w, k, n_embd, part, cpu_part, cpu_flag, sh_out, out, n4, a, mi, seq);
    return note_launch("moe_win_combine_ar");
}

// moe_win_experts; with `ar` the cross-rank sum of out[T][n_embd] (contiguous) runs inside the combine launch.
bool window_down_stream_supported(int d_type, int T, int n_ff);
int window_down_stream(int d_type, const maya_moe_win* w, cudaStream_t s);
int win_experts(int gu_type, int d_type, const maya_moe_win* w, const maya_peer_ar* ar, int mi, unsigned seq, cudaStream_t s) {
    if (!w || !w->plan_w || !w->xq || !w->hq || !w->part || !w->out) return refuse(MAYA_ERR_ARG);
    if (w->cpu_flag != nullptr && w->cpu_part == nullptr) return refuse(MAYA_ERR_ARG);
    int st = check_shapes(gu_type, d_type, w->k, w->n_embd, w->n_ff);
    if (st != MAYA_OK) return refuse(st);
    if (ar != nullptr && (w->out_stride != (size_t) w->n_embd || w->n_embd % 4 || !aligned16(w->out) || !aligned16(w->part) ||
                          (w->sh_out && !aligned16(w->sh_out)) || (w->cpu_part && !aligned16(w->cpu_part))))
        return refuse(MAYA_ERR_ARG);
    st = maya_moe_win_group(w, s);
    if (st != MAYA_OK) return st;
    const int cap = w->T * 8;
    const size_t up_off = row_bytes(gu_type, w->n_embd) * (size_t) w->n_ff;
    // entry id i = t * 8 + j: token t's column (xq_stride apart), h / partial slot i
    GroupArgs A{};
    A.ptr = w->grp_ptr;
    A.start = w->grp_start;
    A.n_groups = w->n_groups;
    A.ent_slot = w->grp_ent;
    A.tok_from_slot = 1;
    st = gate_up_groups(gu_type, A, cap, w->n_embd, w->n_ff, up_off, w->limit, w->xq, w->xq_stride, w->hq, nullptr, 0,
                        nullptr, 0, nullptr, s);
    if (st != MAYA_OK) return st;
    // the down rows streamed through shared memory where the shape allows (moe_window.cu), else read in place
    st = window_down_stream_supported(d_type, w->T, w->n_ff) ? window_down_stream(d_type, w, s)
                                                              : down_groups(d_type, A, cap, w->n_embd, w->n_ff, w->down_off, w->hq, w->part, s);
    if (st != MAYA_OK) return st;
    if (ar != nullptr)
        return win_combine_ar(w->plan_ptr, w->plan_w, w->T, w->k, w->n_embd, w->part, w->cpu_part, w->cpu_flag, w->sh_out, w->out,
                              *ar, mi, seq, s);
    return win_combine(w->plan_ptr, w->plan_w, w->T, w->k, w->n_embd, w->part, w->cpu_part, w->cpu_flag, w->sh_out, w->out,
                       w->out_stride, s);
}

}  // namespace maya

using namespace maya;

extern "C" int maya_moe_gate_up(int gu_type, const maya_moe_plan* plan, int k, int n_embd, int n_ff, float limit,
                                const void* xq, void* hq, const void* sh_down, int sh_type, const void* sh_hq,
                                int n_ff_sh, float* sh_out, void* stream) {
    if (!plan || !plan->plan_ptr || !xq || !hq) return refuse(MAYA_ERR_ARG);
    const int st = check_shapes(gu_type, -1, k, n_embd, n_ff);
    if (st != MAYA_OK) return refuse(st);
    if (sh_down != nullptr) {
        if (!type_is_core(sh_type)) return refuse(MAYA_ERR_TYPE);      // the shared expert's rows: Q8_0, Q4_K, IQ2_S, IQ3_S
        if (!sh_hq || !sh_out || n_ff_sh <= 0 || n_ff_sh % type_qk(sh_type) || n_ff_sh % 32) return refuse(MAYA_ERR_ARG);
    }
    GroupArgs A{};
    A.ptr = plan->plan_ptr;
    A.skip = plan->skip;
    const size_t up_off = row_bytes(gu_type, n_embd) * (size_t) n_ff;
    return gate_up_groups(gu_type, A, k, n_embd, n_ff, up_off, limit, xq, 0, hq, sh_down, sh_type, sh_hq, n_ff_sh, sh_out,
                          as_stream(stream));
}

extern "C" int maya_moe_down(int d_type, const maya_moe_plan* plan, int k, int n_embd, int n_ff, size_t down_off,
                             const void* hq, const float* sh_out, float* out, void* stream) {
    if (!plan || !plan->plan_ptr || !plan->plan_w || !hq || !out) return refuse(MAYA_ERR_ARG);
    if (plan->cpu_flag != nullptr && plan->cpu_part == nullptr) return refuse(MAYA_ERR_ARG);
    const int st = check_shapes(-1, d_type, k, n_embd, n_ff);
    if (st != MAYA_OK) return refuse(st);
    return down_plan(d_type, *plan, k, n_embd, n_ff, down_off, hq, sh_out, out, as_stream(stream));
}

extern "C" int maya_moe_win_group(const maya_moe_win* w, void* stream) {
    if (!w || !w->plan_ptr || !w->grp_ptr || !w->grp_start || !w->grp_ent || !w->n_groups) return refuse(MAYA_ERR_ARG);
    if (w->T < 1 || w->T > MAYA_MAX_WIN_TOKENS || w->k < 1 || w->k > MAYA_MAX_K) return refuse(MAYA_ERR_LIMIT);
    win_group_kernel<<<1, 128, 0, as_stream(stream)>>>(w->plan_ptr, w->T, w->k, w->grp_ptr, w->grp_start, w->grp_ent,
                                                       w->n_groups);
    return note_launch("moe_win_group");
}

extern "C" int maya_moe_win_experts(int gu_type, int d_type, const maya_moe_win* w, void* stream) {
    return win_experts(gu_type, d_type, w, nullptr, 0, 0u, as_stream(stream));
}

extern "C" size_t maya_expert_scratch_bytes(int64_t cap_entries, int64_t n_ff) {
    if (cap_entries <= 0 || n_ff <= 0 || n_ff % 32) return 0;
    return (size_t) cap_entries * (size_t) (n_ff / 32) * kQ81Bytes;   // q8_1 of h per entry; gate/up never leave the SM
}

extern "C" int maya_expert_grouped(const maya_expert_layout* L, const unsigned long long* grp_ptr,
                                   const int32_t* grp_start, const int32_t* n_groups, const int32_t* ent_dst,
                                   const int32_t* ent_tok, int64_t cap_groups, int64_t cap_entries, const void* x_q8_1,
                                   void* scratch, float* out, void* stream, float swiglu_limit) {
    if (!L || !grp_ptr || !grp_start || !n_groups || !ent_dst || !ent_tok || !x_q8_1 || !scratch || !out)
        return refuse(MAYA_ERR_ARG);
    if (cap_groups <= 0 || cap_entries <= 0) return MAYA_OK;
    if (cap_groups > 65535) return refuse(MAYA_ERR_LIMIT);
    if (!type_qk(L->gu_type) || !type_qk(L->d_type)) return refuse(MAYA_ERR_TYPE);
    if (L->n_embd <= 0 || L->n_ff <= 0 || L->n_ff % 32 || L->n_embd % type_qk(L->gu_type) || L->n_ff % type_qk(L->d_type))
        return refuse(MAYA_ERR_ARG);
    cudaStream_t s = as_stream(stream);
    const int n_embd = (int) L->n_embd, n_ff = (int) L->n_ff;
    // entry e: activation column ent_tok[e], h slot e (scratch is per entry), output row ent_dst[e]
    GroupArgs A{};
    A.ptr = grp_ptr;
    A.start = grp_start;
    A.n_groups = n_groups;
    A.ent_tok = ent_tok;
    A.ent_out = ent_dst;
    A.cap_entries = (int) (cap_entries < 0x7fffffff ? cap_entries : 0x7fffffff);   // the scratch (and `out`) hold this many
    const int u_type = L->u_type;                                      // a mixed layer: the up rows' own type (iq_kernels.hpp:73-77)
    if (!type_qk(u_type) || L->n_embd % type_qk(u_type)) return refuse(MAYA_ERR_TYPE);
    int st = u_type == L->gu_type
                 ? gate_up_groups(L->gu_type, A, (int) cap_groups, n_embd, n_ff, L->up_off, swiglu_limit, x_q8_1,
                                  (size_t) (n_embd / 32) * kQ81Bytes, scratch, nullptr, 0, nullptr, 0, nullptr, s)
                 : gate_up_groups_mixed(L->gu_type, u_type, A, (int) cap_groups, n_embd, n_ff, L->up_off, swiglu_limit, x_q8_1,
                                        (size_t) (n_embd / 32) * kQ81Bytes, scratch, s);
    if (st != MAYA_OK) return st;
    return down_groups(L->d_type, A, (int) cap_groups, n_embd, n_ff, L->down_off, scratch, out, s);
}

// ------------------------------------------------------------------------------------------------ no-allocation variant
// Scratch for maya_expert_grouped_static lives in the library image itself: a fixed device array, present on every GPU
// that loads the library for as long as the process lives.  In host code the array's name is only a handle; the
// device address the kernels need comes from cudaGetSymbolAddress, asked once per device with that device current.
constexpr size_t kStaticScratchBytes = (size_t) 2 << 20;
static __device__ __align__(256) unsigned char g_expert_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void* g_static_ptr[kMaxDevices] = {};

// The device address of g_expert_static_scratch on the current device (nullptr + status on failure).
int static_scratch(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return MAYA_ERR_DEVICE; }
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (g_static_ptr[dev] == nullptr) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_expert_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            std::fprintf(stderr, "maya_moe: cudaGetSymbolAddress(static scratch): %s\n", cudaGetErrorString(e));
            cudaGetLastError();
            return MAYA_ERR_LAUNCH;
        }
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return MAYA_OK;
}
}  // namespace

extern "C" size_t maya_expert_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int maya_expert_grouped_static(const maya_expert_layout* L, const unsigned long long* grp_ptr,
                                          const int32_t* grp_start, const int32_t* n_groups, const int32_t* ent_dst,
                                          const int32_t* ent_tok, int64_t cap_groups, int64_t cap_entries,
                                          const void* x_q8_1, float* out, void* stream, float swiglu_limit) {
    if (!L) return refuse(MAYA_ERR_ARG);
    const size_t need = maya_expert_scratch_bytes(cap_entries, L->n_ff);
    if (cap_entries > 0 && need == 0) return refuse(MAYA_ERR_ARG);
    if (need > kStaticScratchBytes) {
        std::fprintf(stderr, "maya_expert_grouped_static: %lld entries of FFN width %lld need %zu bytes of scratch, the "
                             "built-in array holds %zu; use maya_expert_grouped with caller scratch\n",
                     (long long) cap_entries, (long long) L->n_ff, need, kStaticScratchBytes);
        return refuse(MAYA_ERR_LIMIT);
    }
    void* scratch = nullptr;
    const int st = static_scratch(&scratch);
    if (st != MAYA_OK) return refuse(st);
    return maya_expert_grouped(L, grp_ptr, grp_start, n_groups, ent_dst, ent_tok, cap_groups, cap_entries, x_q8_1, scratch,
                               out, stream, swiglu_limit);
}

extern "C" int maya_moe_combine(const float* parts, const float* weights, const float* shared, float* y, int64_t n_embd,
                                int64_t k, int n_tok, void* stream) {
    if (n_tok <= 0) return MAYA_OK;
    if (!parts || !weights || !y || n_embd <= 0) return refuse(MAYA_ERR_ARG);
    if (k < 1 || k > 15) return refuse(MAYA_ERR_LIMIT);
    const dim3 grid((unsigned) ((n_embd + 255) / 256), (unsigned) n_tok);
    combine_kernel<<<grid, 256, 0, as_stream(stream)>>>(parts, weights, shared, y, n_embd, (int) k);
    return note_launch("moe_combine");
}
