// prefill_glue.cu - the prompt path's grouping and glue around the grouped expert GEMM.
//
// Reference entry points replaced (src/kernels/cuda/glm_batch.cu:2102-2215, include/strata/kernels/glm_batch.hpp:131-154):
// expert_count (counts per expert + the stable rank of every routed (token, slot) pair), expert_scatter (sorted row of
// every pair, token of every sorted row), swiglu_rows, moe_combine / moe_combine_add.  The reference copies the counts
// to pinned host memory and builds the per-expert bases on the host (src/core/glm_prefill.cu:3239-3255); here
// maya_expert_bounds does the exclusive scan on the device so the sequence needs no host round trip.
#include <math.h>

#include "maya_common.cuh"
#include "maya_peer_ar.cuh"

namespace maya {
namespace {

// One block per expert.  Warp w owns the pairs [w * per, (w + 1) * per) (per a multiple of 32): a first walk counts its
// pairs routed to this expert, the warps' totals meet in shared memory once, a second walk writes the ranks - a pair's
// rank is the number of earlier pairs routed to the same expert (ballot + popcount inside a warp).
__global__ void __launch_bounds__(1024) expert_count_kernel(const int* __restrict__ ids, int n, int* __restrict__ counts,
                                                            int* __restrict__ rank) {
    const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __shared__ int s_wc[32];
    const int per = ((n + 1023) / 1024) * 32;
    const int i0 = warp * per, i1 = min(n, i0 + per);
    int cnt = 0;
#pragma unroll 4
    for (int i = i0 + lane; i < i1; i += 32) cnt += ids[i] == e;
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    if (lane == 0) s_wc[warp] = cnt;
    __syncthreads();
    int base = 0, tot = 0;
    for (int w = 0; w < 32; ++w) {
        const int c = s_wc[w];
        if (w < warp) base += c;
        tot += c;
    }
    if (cnt != 0) {                                   // warp-uniform: nothing to rank otherwise
        for (int c0 = i0; c0 < i1; c0 += 32) {        // whole warps walk (i0 and per are multiples of 32)
            const int i = c0 + lane;
            const bool m = i < i1 && ids[i] == e;
            const unsigned ballot = __ballot_sync(0xffffffffu, m);
            if (m) rank[i] = base + __popc(ballot & ((1u << lane) - 1u));
            base += __popc(ballot);
        }
    }
    if (tid == 0) counts[e] = tot;
}

// bounds[0] = 0, bounds[e + 1] = bounds[e] + counts[e]; one block.
__global__ void __launch_bounds__(1024) expert_bounds_kernel(const int* __restrict__ counts, int n_expert,
                                                             int* __restrict__ bounds) {
    __shared__ int s_part[1024];
    const int tid = threadIdx.x, per = (n_expert + 1023) / 1024;
    int local = 0;
    for (int j = 0; j < per; ++j) {
        const int e = tid * per + j;
        if (e < n_expert) local += counts[e];
    }
    s_part[tid] = local;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {       // inclusive scan of the per-thread totals
        const int v = tid >= o ? s_part[tid - o] : 0;
        __syncthreads();
        s_part[tid] += v;
        __syncthreads();
    }
    int run = s_part[tid] - local;
    if (tid == 0) bounds[0] = 0;
    for (int j = 0; j < per; ++j) {
        const int e = tid * per + j;
        if (e < n_expert) { run += counts[e]; bounds[e + 1] = run; }
    }
}

__global__ void __launch_bounds__(256) expert_scatter_kernel(const int* __restrict__ ids, const int* __restrict__ rank,
                                                             const int* __restrict__ base, int n, int k,
                                                             int* __restrict__ row_tok, int* __restrict__ pos) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int row = base[ids[i]] + rank[i];
    row_tok[row] = i / k;
    pos[i] = row;
}

// h[r][c] = silu(min(g, L)) * clamp(u, +-L) over rows of [gate | up]; h may alias gu (ld_h = 2 n_ff).
__global__ void __launch_bounds__(256) swiglu_rows_kernel(const float* gu, float* h, int64_t total, int n_ff, int ld_h,
                                                          float limit) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int64_t r = i / n_ff;
    const int c = (int) (i - r * n_ff);
    const float* row = gu + r * 2 * n_ff;
    h[r * ld_h + c] = swiglu(row[c], row[n_ff + c], limit);
}

// ffn[t] = sum_j w[t][j] * out[pos[t][j]] (plan order, m = 0 then m += w * o as the reference's loop) + sh[t]
__global__ void __launch_bounds__(256) combine_rows_kernel(const float* __restrict__ out, const int* __restrict__ pos,
                                                           const float* __restrict__ w, const float* __restrict__ sh,
                                                           int k, int n_embd, float* __restrict__ ffn) {
    const int t = blockIdx.y, e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n_embd) return;
    float m = 0.0f;
    for (int j = 0; j < k; ++j) m = __fmaf_rn(w[t * k + j], out[(size_t) pos[t * k + j] * n_embd + e], m);
    ffn[(size_t) t * n_embd + e] = __fadd_rn(m, sh ? sh[(size_t) t * n_embd + e] : 0.0f);
}
// the same, four columns a thread (n_embd % 4 == 0, 16-byte aligned rows): the k rows' loads are issued together
template<int K>
__global__ void __launch_bounds__(256) combine_rows4_kernel(const float* __restrict__ out, const int* __restrict__ pos,
                                                            const float* __restrict__ w, const float* __restrict__ sh,
                                                            int k, int n_embd, float* __restrict__ ffn) {
    const int t = blockIdx.y, e = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (e >= n_embd) return;
    const int kk = K > 0 ? K : k;
    float4 m = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if constexpr (K > 0) {
        float4 o[K];
        float wj[K];
#pragma unroll
        for (int j = 0; j < K; ++j) {
            wj[j] = w[t * K + j];
            o[j] = __ldcs((const float4*) (out + (size_t) pos[t * K + j] * n_embd + e));
        }
#pragma unroll
        for (int j = 0; j < K; ++j) {
            m.x = __fmaf_rn(wj[j], o[j].x, m.x); m.y = __fmaf_rn(wj[j], o[j].y, m.y);
            m.z = __fmaf_rn(wj[j], o[j].z, m.z); m.w = __fmaf_rn(wj[j], o[j].w, m.w);
        }
    } else {
        for (int j = 0; j < kk; ++j) {
            const float wj = w[t * kk + j];
            const float4 o = __ldcs((const float4*) (out + (size_t) pos[t * kk + j] * n_embd + e));
            m.x = __fmaf_rn(wj, o.x, m.x); m.y = __fmaf_rn(wj, o.y, m.y); m.z = __fmaf_rn(wj, o.z, m.z); m.w = __fmaf_rn(wj, o.w, m.w);
        }
    }
    float4 s4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (sh) s4 = *(const float4*) (sh + (size_t) t * n_embd + e);
    m.x = __fadd_rn(m.x, s4.x); m.y = __fadd_rn(m.y, s4.y); m.z = __fadd_rn(m.z, s4.z); m.w = __fadd_rn(m.w, s4.w);
    *(float4*) (ffn + (size_t) t * n_embd + e) = m;
}

// the same over this rank's experts only: a route whose expert id is outside [e_lo, e_hi) contributes an exact zero
// (its sorted row was never computed here); the ranks' results add up to combine_rows_kernel's
__global__ void __launch_bounds__(256) combine_rows_local_kernel(const float* __restrict__ out, const int* __restrict__ pos,
                                                                 const float* __restrict__ w, const int* __restrict__ ids,
                                                                 int e_lo, int e_hi, const float* __restrict__ sh, int k,
                                                                 int n_embd, float* __restrict__ ffn) {
    const int t = blockIdx.y, e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n_embd) return;
    float m = 0.0f;
    for (int j = 0; j < k; ++j) {
        const int id = ids[t * k + j];
        if (id >= e_lo && id < e_hi) m = __fmaf_rn(w[t * k + j], out[(size_t) pos[t * k + j] * n_embd + e], m);
    }
    ffn[(size_t) t * n_embd + e] = __fadd_rn(m, sh ? sh[(size_t) t * n_embd + e] : 0.0f);
}

// combine_rows_local_kernel and the cross-rank sum in one launch: block b combines its share [q0, q1) (float4 units of
// the flat [T][n_embd] result) into ffn, then pushes it to every peer's receive slot, raises its flag there, waits
// (bounded) for the peers' flags and adds the nm rows in rank order (peer_allreduce_block: the rows + flags form).
__global__ void __launch_bounds__(256) combine_rows_local_ar_kernel(const float* __restrict__ out, const int* __restrict__ pos,
                                                                    const float* __restrict__ w, const int* __restrict__ ids,
                                                                    int e_lo, int e_hi, const float* __restrict__ sh, int k,
                                                                    int n_embd, float* ffn, int n4, maya_peer_ar a, int mi,
                                                                    unsigned seq) {
    const int nb = gridDim.x, b = blockIdx.x;
    const int base = n4 / nb, rem = n4 % nb;
    const int q0 = b * base + min(b, rem), q1 = q0 + base + (b < rem ? 1 : 0);
    for (int q = q0 + threadIdx.x; q < q1; q += blockDim.x) {
        const int t = (int) (((size_t) q * 4) / n_embd), e = (int) ((size_t) q * 4 - (size_t) t * n_embd);
        float4 m = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int j = 0; j < k; ++j) {
            const int id = ids[t * k + j];
            if (id >= e_lo && id < e_hi) {
                const float wj = w[t * k + j];
                const float4 o = *(const float4*) (out + (size_t) pos[t * k + j] * n_embd + e);
                m.x = __fmaf_rn(wj, o.x, m.x); m.y = __fmaf_rn(wj, o.y, m.y); m.z = __fmaf_rn(wj, o.z, m.z); m.w = __fmaf_rn(wj, o.w, m.w);
            }
        }
        float4 s4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (sh) s4 = *(const float4*) (sh + (size_t) t * n_embd + e);
        m.x = __fadd_rn(m.x, s4.x); m.y = __fadd_rn(m.y, s4.y); m.z = __fadd_rn(m.z, s4.z); m.w = __fadd_rn(m.w, s4.w);
        ((float4*) ffn)[q] = m;
    }
    __syncthreads();
    const unsigned sq = ar_seq_begin(a, seq);
    peer_allreduce_block(ffn, q0, q1, a, mi, sq, b);
    ar_seq_end(a, seq, sq);
}

// ffn[t] += sum over t's routes whose sorted row lies in [lo, hi) of w * out[row - base]
__global__ void __launch_bounds__(256) combine_add_kernel(const float* __restrict__ out, int base, int lo, int hi,
                                                          const int* __restrict__ pos, const float* __restrict__ w, int k,
                                                          int n_embd, float* __restrict__ ffn) {
    const int t = blockIdx.y, e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n_embd) return;
    float m = 0.0f;
    bool any = false;
    for (int j = 0; j < k; ++j) {
        const int p = pos[t * k + j];
        if (p >= lo && p < hi) { m = __fmaf_rn(w[t * k + j], out[(size_t) (p - base) * n_embd + e], m); any = true; }
    }
    if (any) ffn[(size_t) t * n_embd + e] = __fadd_rn(ffn[(size_t) t * n_embd + e], m);
}

}  // namespace
}  // namespace maya

using namespace maya;

extern "C" int maya_expert_count(const int* ids, int n, int n_expert, int* counts, int* rank, void* stream) {
    if (n_expert <= 0) return MAYA_OK;
    if (!counts || n < 0 || (n > 0 && (!ids || !rank))) return refuse(MAYA_ERR_ARG);
    expert_count_kernel<<<n_expert, 1024, 0, as_stream(stream)>>>(ids, n, counts, rank);
    return note_launch("expert_count");
}
extern "C" int maya_expert_bounds(const int* counts, int n_expert, int* bounds, void* stream) {
    if (!counts || !bounds || n_expert <= 0) return refuse(MAYA_ERR_ARG);
    expert_bounds_kernel<<<1, 1024, 0, as_stream(stream)>>>(counts, n_expert, bounds);
    return note_launch("expert_bounds");
}
extern "C" int maya_expert_scatter(const int* ids, const int* rank, const int* base, int n, int k, int* row_tok, int* pos,
                                   void* stream) {
    if (n <= 0) return MAYA_OK;
    if (!ids || !rank || !base || !row_tok || !pos || k <= 0) return refuse(MAYA_ERR_ARG);
    expert_scatter_kernel<<<(n + 255) / 256, 256, 0, as_stream(stream)>>>(ids, rank, base, n, k, row_tok, pos);
    return note_launch("expert_scatter");
}
extern "C" int maya_swiglu_rows(const float* gu, float* h, int rows, int n_ff, float limit, int ld_h, void* stream) {
    if (rows <= 0) return MAYA_OK;
    if (!gu || !h || n_ff <= 0 || ld_h < 0) return refuse(MAYA_ERR_ARG);
    const int64_t total = (int64_t) rows * n_ff;
    swiglu_rows_kernel<<<(unsigned) ((total + 255) / 256), 256, 0, as_stream(stream)>>>(gu, h, total, n_ff,
                                                                                       ld_h ? ld_h : n_ff, limit);
    return note_launch("swiglu_rows");
}
extern "C" int maya_moe_combine_rows(const float* out, const int* pos, const float* w, const float* sh, int T, int k,
                                     int n_embd, float* ffn, void* stream) {
    if (T <= 0) return MAYA_OK;
    if (!out || !pos || !w || !ffn || k <= 0 || n_embd <= 0) return refuse(MAYA_ERR_ARG);
    if (n_embd % 4 == 0 && aligned16(out) && aligned16(ffn) && (!sh || aligned16(sh))) {
        const dim3 grid4((unsigned) ((n_embd / 4 + 255) / 256), (unsigned) T);
        if (k == 8) combine_rows4_kernel<8><<<grid4, 256, 0, as_stream(stream)>>>(out, pos, w, sh, k, n_embd, ffn);
        else combine_rows4_kernel<0><<<grid4, 256, 0, as_stream(stream)>>>(out, pos, w, sh, k, n_embd, ffn);
        return note_launch("moe_combine_rows");
    }
    const dim3 grid((unsigned) ((n_embd + 255) / 256), (unsigned) T);
    combine_rows_kernel<<<grid, 256, 0, as_stream(stream)>>>(out, pos, w, sh, k, n_embd, ffn);
    return note_launch("moe_combine_rows");
}
extern "C" int maya_moe_combine_rows_local(const float* out, const int* pos, const float* w, const int* ids, int e_lo,
                                           int e_hi, const float* sh, int T, int k, int n_embd, float* ffn, void* stream) {
    if (T <= 0) return MAYA_OK;
    if (!out || !pos || !w || !ids || !ffn || k <= 0 || n_embd <= 0 || e_lo > e_hi) return refuse(MAYA_ERR_ARG);
    const dim3 grid((unsigned) ((n_embd + 255) / 256), (unsigned) T);
    combine_rows_local_kernel<<<grid, 256, 0, as_stream(stream)>>>(out, pos, w, ids, e_lo, e_hi, sh, k, n_embd, ffn);
    return note_launch("moe_combine_rows_local");
}
extern "C" int maya_moe_combine_rows_local_ar(const float* out, const int* pos, const float* w, const int* ids, int e_lo,
                                              int e_hi, const float* sh, int T, int k, int n_embd, float* ffn,
                                              const maya_peer_ar* a, int mi, unsigned seq, void* stream) {
    if (T <= 0) return MAYA_OK;
    if (!out || !pos || !w || !ids || !ffn || k <= 0 || n_embd <= 0 || n_embd % 4 || e_lo > e_hi) return refuse(MAYA_ERR_ARG);
    if (!a || !a->recv || !a->peer_recv || !a->flags || !a->peer_flags || !a->error || a->timeout_ns == 0) return refuse(MAYA_ERR_ARG);
    if (a->nm < 2 || a->nm > MAYA_PEER_AR_MAX_RANKS || mi < 0 || mi >= a->nm || a->stride % 4) return refuse(MAYA_ERR_ARG);
    if (seq == 0u && a->seq_counter == nullptr) return refuse(MAYA_ERR_ARG);
    if ((size_t) T * n_embd > a->stride || !aligned16(ffn) || !aligned16(out) || (sh && !aligned16(sh))) return refuse(MAYA_ERR_ARG);
    const int n4 = (int) ((size_t) T * n_embd / 4);
    int blocks = (n4 + 255) / 256;
    if (blocks > MAYA_PEER_AR_BLOCKS) blocks = MAYA_PEER_AR_BLOCKS;
    combine_rows_local_ar_kernel<<<blocks, 256, 0, as_stream(stream)>>>(out, pos, w, ids, e_lo, e_hi, sh, k, n_embd, ffn, n4, *a,
                                                                        mi, seq);
    return note_launch("moe_combine_rows_local_ar");
}
extern "C" int maya_moe_combine_add(const float* out, int base, int lo, int hi, const int* pos, const float* w, int T,
                                    int k, int n_embd, float* ffn, void* stream) {
    if (T <= 0 || hi <= lo) return MAYA_OK;
    if (!out || !pos || !w || !ffn || k <= 0 || n_embd <= 0) return refuse(MAYA_ERR_ARG);
    const dim3 grid((unsigned) ((n_embd + 255) / 256), (unsigned) T);
    combine_add_kernel<<<grid, 256, 0, as_stream(stream)>>>(out, base, lo, hi, pos, w, k, n_embd, ffn);
    return note_launch("moe_combine_add");
}
