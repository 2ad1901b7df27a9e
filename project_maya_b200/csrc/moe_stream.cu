// moe_stream.cu - one token through one MoE layer in ONE persistent kernel whose weight rows are streamed through
// shared memory by the TMA engine (maya_stream.cuh): route, quantize the activation, routed and shared gate/up +
// SwiGLU, q8_1 of h, routed and shared down, weighted combine, cross-rank sum, residual write.
//
// Same result bits as the grid-barrier kernel of moe_fused.cu and as the staged kernels; what differs is the schedule:
//   * nothing waits for the router that does not need it: warps 0-7 quantize x and start on the shared expert's gate/up
//     rows (Q8_0: 29 % of the layer's bytes, almost no arithmetic) while warps 8-15 route;
//   * no grid barrier.  Gate/up work is (expert slot, two FFN rows) items dealt to the blocks in equal shares; a 32-row
//     unit of h is rounded to q8_1 by whichever warp, of whichever block, completes it (a counter per unit), and the
//     down rows of an expert slot wait only for that slot's units (a counter per slot).  A block that runs out of gate/up
//     items goes on with the shared expert's down rows and the slots that are already complete;
//   * a block's warps take their items from two queues in shared memory (gate/up, then down), so a warp that joins late
//     (the routing warps) or draws longer items does not hold the block up;
//   * the rows come in by bulk copies into a two-slot ring per warp: no load instructions, address arithmetic or
//     scoreboard stalls in the dot loops, and the shared expert streams at HBM rate under the integer-bound i-quant work.
//
// Every wait is bounded; one that runs out sets the sticky error word of the scratch and the block's `fail` flag, after
// which the block stops computing, waits (bounded) for its copies in flight and runs to its end.
#include "maya_stream.cuh"
#include "maya_internal.cuh"
#include "maya_peer_ar.cuh"
#include "maya_hc_post.cuh"
#include "maya_router.cuh"
#include "maya_fused_args.cuh"

#include <atomic>

namespace maya {
namespace {

constexpr int kSThreads = 512;
constexpr int kDotWarps = 12;             // warps 0..11 run the dot loops
constexpr int kXWarps = 8;                // warps 0..7 quantize x
constexpr int kRouteThreads = 256;        // warps 8..15 route
constexpr int kHelpThreads = 128;         // warps 12..15: bring each slot's q8_1(h) into shared memory as it completes
constexpr int kSlots = 2;
constexpr int kMaxRows = 64;              // output rows a block may own
constexpr unsigned kSpin = 1u << 22;
constexpr int kSlotsMax = MAYA_MAX_K + 1;

struct StreamShared {
    RouterShared route;
    unsigned long long ptr[kSlotsMax];
    float w[MAYA_MAX_K];
    int ve[MAYA_MAX_K];
    int nv;
    float part[kMaxRows][kSlotsMax];
    uint64_t bar_ring[kDotWarps * kSlots];
    uint64_t bar_plan, bar_x;
    uint64_t bar_h[kSlotsMax];
    int qa, qb;
    int ra0, nra;                          // this block's share of the routed gate/up items
    unsigned ar_seq;
    int fail;
};

// the kernel's part of the caller's scratch (FusedArgs::h), all of it zero between launches except hf / gq / gd
struct StreamScratch {
    float* hf;          // [9][h_ld] f32 h
    int8_t* gq;         // [9][h_ld] q8_1 quants of h
    float* gd;          // [9][h_ld / 32] their scales
    unsigned* ucnt;     // [9][h_ld / 32] items arrived per 32-row unit
    unsigned* ecnt;     // [9] units completed per slot; [15]: blocks done
};
__host__ __device__ inline StreamScratch stream_scratch(float* h, int h_ld) {
    StreamScratch s;
    const int nb = h_ld / 32;
    s.hf = h;
    s.gq = (int8_t*) (h + (size_t) kSlotsMax * h_ld);
    s.gd = (float*) (s.gq + (size_t) kSlotsMax * h_ld);
    s.ucnt = (unsigned*) (s.gd + (size_t) kSlotsMax * nb);
    s.ecnt = s.ucnt + (size_t) kSlotsMax * nb;
    return s;
}

__device__ __forceinline__ unsigned long long s_global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void s_stamp(unsigned* sync, int i) {
    *(volatile unsigned long long*) &sync[4 + 2 * i] = s_global_ns();
}
__device__ __forceinline__ void s_slice(int n, int nb, int b, int& r0, int& r1) {
    const int base = n / nb, rem = n % nb;
    r0 = b * base + min(b, rem);
    r1 = r0 + base + (b < rem ? 1 : 0);
}
__device__ __forceinline__ void mbar_arrive1(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// item kinds
enum { kQA = 0, kIA = 1, kQB = 2, kIB = 3 };
// packed item + stage: kind (2) | slot (4) | seg (3) | last-seg flag (1) | r (22)
__device__ __forceinline__ int pack_stage(int kind, int slot, int seg, int last, int r) {
    return kind | (slot << 2) | (seg << 6) | (last << 9) | (r << 10);
}

template<int T> struct IqDot;
template<> struct IqDot<MAYA_IQ2_S> {
    __device__ __forceinline__ static void stage(const uint8_t* st, const uint8_t* ximg_seg, const uint32_t* tab, int lane, float (&acc)[4]) {
        iq2s_stage<false, 16>(st, ximg_seg, (const uint2*) tab + (lane & 15), lane, acc);
    }
};

template<int T, int TS>
__global__ void __launch_bounds__(kSThreads, 1) moe_layer_t1_stream_kernel(FusedArgs A) {
    extern __shared__ __align__(128) uint8_t s_raw[];
    __shared__ StreamShared sh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int k = A.k, n_embd = A.n_embd, n_ff = A.n_ff;
    const bool has_sh = TS != 0 && A.shared != nullptr;
    const int n_ff_sh = has_sh ? A.n_ff_sh : 0;
    const int h_ld = max(n_ff, A.n_ff_sh);
    const int nblk_x = n_embd / 32, nblk_h = h_ld / 32;
    constexpr int kSlotBytes = (Stage<T>::bytes > Stage<MAYA_Q8_0>::bytes ? Stage<T>::bytes : Stage<MAYA_Q8_0>::bytes);

    // shared memory: [replicated codebook | image of x | images of h, one per slot | ring | router scratch]
    uint32_t* s_tab = (uint32_t*) s_raw;
    uint8_t* ximg = s_raw + kRepTabBytes<T>;
    uint8_t* himg = ximg + ximg_bytes(nblk_x);
    const size_t himg_slot = ximg_bytes(nblk_h);
    uint8_t* ring = himg + (size_t) kSlotsMax * himg_slot;
    double* s_ex = (double*) (ring + (size_t) kDotWarps * kSlots * kSlotBytes);
    const StreamScratch G = stream_scratch(A.h, h_ld);

    // Programmatic dependent launch: nothing of global memory is touched before griddepcontrol.wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    load_tab_rep<T>(s_tab, tid, kSThreads);
    if (tid == 0) {
        for (int i = 0; i < kDotWarps * kSlots; ++i) mbar_init(&sh.bar_ring[i], 1);
        mbar_init(&sh.bar_plan, 1);
        mbar_init(&sh.bar_x, 1);
        for (int i = 0; i < kSlotsMax; ++i) mbar_init(&sh.bar_h[i], 1);
        sh.qa = 0; sh.qb = 0; sh.fail = 0; sh.nv = 0; sh.ra0 = 0; sh.nra = 0;
    }
    mbar_fence_init();
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) {
        sh.ar_seq = A.ar_seq != 0u || A.ar.seq_counter == nullptr ? A.ar_seq : *(volatile unsigned*) A.ar.seq_counter + 1u;
        if (blockIdx.x == 0) s_stamp(A.sync, 0);
    }
    __syncthreads();

    // this block's shares: gate/up items of the shared expert (one FFN row each), output rows (whole quads)
    int sa0, sa1, o0, o1;
    s_slice(n_ff_sh, gridDim.x, blockIdx.x, sa0, sa1);
    s_slice(n_embd / 4, gridDim.x, blockIdx.x, o0, o1);
    o0 *= 4;
    o1 *= 4;
    const int nrows = o1 - o0, nsa = sa1 - sa0, ns2 = has_sh ? nrows / 2 : 0;
    const size_t rb = row_bytes(T, n_embd), drb = row_bytes(T, n_ff), down_off = 2 * (size_t) n_ff * rb;
    const size_t rbs = row_bytes(MAYA_Q8_0, n_embd), drbs = row_bytes(MAYA_Q8_0, A.n_ff_sh);
    const uint8_t* sh_down = has_sh ? A.shared + 2 * (size_t) A.n_ff_sh * rbs : nullptr;

    if (warp >= kXWarps) {
        // ------------------------------------------------------------ routing (warps 8-15)
        const int t = tid - kXWarps * 32;
        using RS = NamedSync<1, kRouteThreads>;
        const int per = (A.n_expert + kRouteThreads - 1) / kRouteThreads;
        if (per <= 1) route_softmax<1, RS>(A.logits, A.n_expert, k, t, kRouteThreads, s_ex, sh.route);
        else if (per <= 2) route_softmax<2, RS>(A.logits, A.n_expert, k, t, kRouteThreads, s_ex, sh.route);
        else if (per <= 4) route_softmax<4, RS>(A.logits, A.n_expert, k, t, kRouteThreads, s_ex, sh.route);
        else route_softmax<8, RS>(A.logits, A.n_expert, k, t, kRouteThreads, s_ex, sh.route);
        if (t < k) {
            const int e = sh.route.ids[t];
            sh.w[t] = sh.route.val[t];
            sh.ptr[t] = (e >= A.expert_lo && e < A.expert_hi) ? (unsigned long long) (A.experts + (size_t) e * A.expert_stride) : 0ull;
            if (blockIdx.x == 0) { A.ids[t] = e; A.weights[t] = sh.route.val[t]; }
        }
        if (t == 0) sh.ptr[k] = has_sh ? (unsigned long long) A.shared : 0ull;
        RS::sync();
        if (t == 0) {
            int nv = 0;
            for (int i = 0; i < k; ++i)
                if (sh.ptr[i] != 0ull) sh.ve[nv++] = i;
            sh.nv = nv;
            int a0, a1;
            s_slice(nv * (n_ff / 2), gridDim.x, blockIdx.x, a0, a1);
            sh.ra0 = a0;
            sh.nra = a1 - a0;
            __threadfence_block();
            mbar_arrive1(&sh.bar_plan);
            if (blockIdx.x == 0) s_stamp(A.sync, 1);
        }
    } else {
        // ------------------------------------------------------------ q8_1(x) into the image (warps 0-7)
        for (int b0 = warp; b0 < nblk_x; b0 += 8 * kXWarps) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int b = b0 + i * kXWarps;
                v[i] = 0.0f;
                if (b < nblk_x)
                    v[i] = A.x_is_bf16 ? __uint_as_float((uint32_t) ((const uint16_t*) A.x)[b * 32 + lane] << 16)
                                       : ((const float*) A.x)[b * 32 + lane];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (b0 + i * kXWarps < nblk_x) ximg_store_warp(v[i], ximg, b0 + i * kXWarps, lane);
        }
        NamedSync<3, kXWarps * 32>::sync();
        if (tid == 0) { __threadfence_block(); mbar_arrive1(&sh.bar_x); }
    }

    if (warp < kDotWarps) {
        // ------------------------------------------------------------ the dot loops (warps 0-11)
        bool ok = true;
        if (warp >= kXWarps) ok = mbar_wait(&sh.bar_x, 0);
        uint8_t* my_ring = ring + (size_t) warp * kSlots * kSlotBytes;
        uint64_t* my_bar = &sh.bar_ring[warp * kSlots];
        // issue cursor
        int c_kind = -1, c_slot = 0, c_r = 0, c_seg = 0, c_nseg = 0, c_queue = 0;
        bool plan_seen = false;
        int nv = 0, nra = 0, ra0 = 0, nr2 = 0;
        const int nseg_qa = n_embd / Stage<MAYA_Q8_0>::seg_vals, nseg_ia = n_embd / Stage<T>::seg_vals;
        const int nseg_qb = has_sh ? A.n_ff_sh / Stage<MAYA_Q8_0>::seg_vals : 0, nseg_ib = n_ff / Stage<T>::seg_vals;
        auto need_plan = [&]() {
            if (!plan_seen) {
                if (!mbar_wait(&sh.bar_plan, 0)) ok = false;
                plan_seen = true;
                nv = sh.nv; nra = sh.nra; ra0 = sh.ra0;
                nr2 = nv * (nrows / 4);
            }
        };
        // the next stage of this warp's work into ring slot `slot`; -1 when there is none
        auto issue_next = [&](int slot) -> int {
            if (!ok) return -1;
            if (c_kind >= 0 && c_seg + 1 < c_nseg) {
                ++c_seg;
            } else {
                c_kind = -1;
                if (c_queue == 0) {
                    int q = 0;
                    if (lane == 0) q = atomicAdd(&sh.qa, 1);
                    q = __shfl_sync(0xffffffffu, q, 0);
                    if (q < nsa) {
                        c_kind = kQA; c_slot = k; c_r = sa0 + q; c_nseg = nseg_qa;
                    } else {
                        need_plan();
                        if (!ok) return -1;
                        if (q - nsa < nra) {
                            const int t = ra0 + (q - nsa), half = n_ff / 2, ei = t / half;
                            c_kind = kIA; c_slot = sh.ve[ei]; c_r = 2 * (t - ei * half); c_nseg = nseg_ia;
                        } else {
                            c_queue = 1;
                        }
                    }
                }
                if (c_queue == 1) {
                    need_plan();
                    if (!ok) return -1;
                    int q = 0;
                    if (lane == 0) q = atomicAdd(&sh.qb, 1);
                    q = __shfl_sync(0xffffffffu, q, 0);
                    if (q < ns2) {
                        c_kind = kQB; c_slot = k; c_r = o0 + 2 * q; c_nseg = nseg_qb;
                    } else if (q - ns2 < nr2) {
                        const int t = q - ns2, quads = nrows / 4, ei = t / quads;
                        c_kind = kIB; c_slot = sh.ve[ei]; c_r = o0 + 4 * (t - ei * quads); c_nseg = nseg_ib;
                    } else {
                        c_queue = 2;
                    }
                }
                if (c_kind < 0) return -1;
                c_seg = 0;
            }
            if (lane == 0) {
                uint8_t* dst = my_ring + slot * kSlotBytes;
                uint64_t* bar = &my_bar[slot];
                if (c_kind == kQA || c_kind == kQB) {
                    using S = Stage<MAYA_Q8_0>;
                    const uint8_t* r0p;
                    const uint8_t* r1p;
                    if (c_kind == kQA) {
                        r0p = A.shared + (size_t) c_r * rbs;
                        r1p = A.shared + (size_t) (A.n_ff_sh + c_r) * rbs;
                    } else {
                        r0p = sh_down + (size_t) c_r * drbs;
                        r1p = r0p + drbs;
                    }
                    const size_t so = (size_t) c_seg * S::seg_bytes;
                    mbar_expect_tx(bar, 2 * S::seg_bytes);
                    bulk_load(dst, r0p + so, S::seg_bytes, bar);
                    bulk_load(dst + S::pitch, r1p + so, S::seg_bytes, bar);
                } else {
                    using S = Stage<T>;
                    const uint8_t* blob = (const uint8_t*) sh.ptr[c_slot];
                    const size_t so = (size_t) c_seg * S::seg_bytes;
                    mbar_expect_tx(bar, 4 * S::seg_bytes);
                    if (c_kind == kIA) {
                        const uint8_t* g0 = blob + (size_t) c_r * rb + so;
                        const uint8_t* u0 = blob + (size_t) (n_ff + c_r) * rb + so;
                        bulk_load(dst, g0, S::seg_bytes, bar);
                        bulk_load(dst + S::pitch, u0, S::seg_bytes, bar);
                        bulk_load(dst + 2 * S::pitch, g0 + rb, S::seg_bytes, bar);
                        bulk_load(dst + 3 * S::pitch, u0 + rb, S::seg_bytes, bar);
                    } else {
                        const uint8_t* d0 = blob + down_off + (size_t) c_r * drb + so;
#pragma unroll
                        for (int g = 0; g < 4; ++g) bulk_load(dst + g * S::pitch, d0 + (size_t) g * drb, S::seg_bytes, bar);
                    }
                }
            }
            return pack_stage(c_kind, c_slot, c_seg, c_seg + 1 == c_nseg, c_r);
        };

        int f0 = issue_next(0);
        int f1 = f0 >= 0 ? issue_next(1) : -1;
        int slot = 0;
        uint32_t phase = 0;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        bool stamped = false;
        while (f0 >= 0) {
            const int kind = f0 & 3, sl = (f0 >> 2) & 15, seg = (f0 >> 6) & 7, last = (f0 >> 9) & 1, r = f0 >> 10;
            if (seg == 0) {
                acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
                if (kind >= kQB) {
                    if (blockIdx.x == 0 && warp == 0 && !stamped) { stamped = true; if (lane == 0) s_stamp(A.sync, 2); }
                    if (ok && !mbar_wait(&sh.bar_h[sl], 0)) ok = false;
                }
            }
            if (ok && !mbar_wait(&my_bar[slot], phase)) ok = false;
            if (ok && *(volatile int*) &sh.fail) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint8_t* st = my_ring + slot * kSlotBytes;
            {
                if (kind == kQA) {
                    float a2[2] = {acc[0], acc[1]};
                    q8_0_stage(st, ximg + (size_t) seg * 8 * kXHalfBytes, lane, a2);
                    acc[0] = a2[0]; acc[1] = a2[1];
                } else if (kind == kQB) {
                    float a2[2] = {acc[0], acc[1]};
                    q8_0_stage(st, himg + (size_t) sl * himg_slot + (size_t) seg * 8 * kXHalfBytes, lane, a2);
                    acc[0] = a2[0]; acc[1] = a2[1];
                } else if (kind == kIA) {
                    IqDot<T>::stage(st, ximg + (size_t) seg * 16 * kXHalfBytes, s_tab, lane, acc);
                } else {
                    IqDot<T>::stage(st, himg + (size_t) sl * himg_slot + (size_t) seg * 16 * kXHalfBytes, s_tab, lane, acc);
                }
            }
            __syncwarp();
            fence_proxy_async();
            const int fn = issue_next(slot);
            if (last) {
                if (kind == kQA || kind == kIA) {
                    float h0, h1 = 0.0f;
                    int per_unit;
                    if (kind == kQA) {
                        const float a2[2] = {acc[0], acc[1]};
                        const float v = q8_0_row_sum(a2);
                        h0 = swiglu(__shfl_sync(0xffffffffu, v, 0), __shfl_sync(0xffffffffu, v, 16), A.limit);
                        per_unit = 32;
                    } else {
                        const float v = iq_row_sum(acc);
                        h0 = swiglu(__shfl_sync(0xffffffffu, v, 0), __shfl_sync(0xffffffffu, v, 8), A.limit);
                        h1 = swiglu(__shfl_sync(0xffffffffu, v, 16), __shfl_sync(0xffffffffu, v, 24), A.limit);
                        per_unit = 16;
                    }
                    const int unit = sl * nblk_h + (r >> 5);
                    unsigned old = 0;
                    if (lane == 0) {
                        G.hf[(size_t) sl * h_ld + r] = h0;
                        if (kind == kIA) G.hf[(size_t) sl * h_ld + r + 1] = h1;
                        __threadfence();
                        old = atomicAdd(&G.ucnt[unit], 1u);
                    }
                    old = __shfl_sync(0xffffffffu, old, 0);
                    if (old == (unsigned) per_unit - 1u) {       // this warp completed the unit: round it to q8_1
                        __threadfence();
                        const float hv = __ldcg(&G.hf[(size_t) sl * h_ld + (r & ~31) + lane]);
                        const float amax = warp_max(fabsf(hv));
                        const float dd = fminf(__fdiv_rn(amax, 127.0f), 65504.0f);
                        const int qi = amax == 0.0f ? 0 : (int) fmaxf(-127.0f, fminf(127.0f, roundf(__fdiv_rn(hv, dd))));
                        G.gq[(size_t) unit * 32 + lane] = (int8_t) qi;
                        if (lane == 0) G.gd[unit] = __half2float(__float2half_rn(dd));
                        __threadfence();
                        __syncwarp();
                        if (lane == 0) {
                            G.ucnt[unit] = 0u;
                            __threadfence();
                            atomicAdd(&G.ecnt[sl], 1u);
                        }
                    }
                } else if (kind == kQB) {
                    const float a2[2] = {acc[0], acc[1]};
                    const float v = q8_0_row_sum(a2);
                    if ((lane & 15) == 0) sh.part[r - o0 + (lane >> 4)][k] = v;
                } else {
                    const float v = iq_row_sum(acc);
                    if ((lane & 7) == 0) sh.part[r - o0 + (lane >> 3)][sl] = v;
                }
            }
            f0 = f1;
            f1 = fn;
            slot ^= 1;
            if (slot == 0) phase ^= 1u;
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
            // gave up: flag it, and let the copies still in flight into this warp's slots land before the block ends
            if (lane == 0) { atomicExch(&sh.fail, 1); atomicExch(&A.sync[2], 1u); }
            if (f0 >= 0) mbar_wait(&my_bar[slot], phase);
            if (f1 >= 0) mbar_wait(&my_bar[slot ^ 1], slot == 1 ? phase ^ 1u : phase);
        }
    } else {
        // ------------------------------------------------------------ helpers (warps 12-15): q8_1(h) of each slot
        const int t = tid - kDotWarps * 32;
        using HS = NamedSync<2, kHelpThreads>;
        const bool planned = mbar_wait(&sh.bar_plan, 0);       // nv and ve are written after the routing group's last barrier
        if (!planned && t == 0) { atomicExch(&sh.fail, 1); atomicExch(&A.sync[2], 1u); }
        const int nv = planned ? sh.nv : 0;
        for (int oi = has_sh && planned ? -1 : 0; oi < nv; ++oi) {
            const int sl = oi < 0 ? k : sh.ve[oi];
            const int nb = (oi < 0 ? A.n_ff_sh : n_ff) / 32;
            if (t == 0) {
                unsigned spins = 0;
                while (*(volatile unsigned*) &G.ecnt[sl] < (unsigned) nb) {
                    if (*(volatile int*) &sh.fail || ++spins > kSpin) { atomicExch(&sh.fail, 1); atomicExch(&A.sync[2], 1u); break; }
                    __nanosleep(40);
                }
                __threadfence();
            }
            HS::sync();
            if (!*(volatile int*) &sh.fail) {
                uint8_t* img = himg + (size_t) sl * himg_slot;
                for (int b = t; b < nb; b += kHelpThreads) {
                    const uint4* src = (const uint4*) (G.gq + ((size_t) sl * nblk_h + b) * 32);
                    uint4* dst = (uint4*) ximg_q(img, b);
                    dst[0] = __ldcg(src);
                    dst[1] = __ldcg(src + 1);
                    *ximg_d(img, b) = __ldcg(&G.gd[(size_t) sl * nblk_h + b]);
                }
            }
            HS::sync();
            if (t == 0) {
                __threadfence_block();
                mbar_arrive1(&sh.bar_h[sl]);
                if (blockIdx.x == 0 && oi == nv - 1) s_stamp(A.sync, 3);
            }
        }
    }
    __syncthreads();
    const bool good = *(volatile int*) &sh.fail == 0;
    if (good && tid < nrows) {
        float m = 0.0f;
        for (int i = 0; i < k; ++i) m = __fmaf_rn(sh.w[i], sh.ptr[i] != 0ull ? sh.part[tid][i] : 0.0f, m);
        A.out[o0 + tid] = __fadd_rn(m, has_sh ? sh.part[tid][k] : 0.0f);
    }
    if (blockIdx.x == 0 && tid == 0) s_stamp(A.sync, 4);
    // ---------------------------------------------------------------- epilogue: the cross-rank sum of this block's rows
    bool summed = good;
    if (A.ar.nm >= 2) {
        __syncthreads();
        if (good) summed = peer_allreduce_block_words(A.out, o0 / 4, o1 / 4, A.ar, A.ar_rank, sh.ar_seq, blockIdx.x);
    }
    __syncthreads();
    if (A.hc.R_new != nullptr && summed) hc_post_rows(A.out, A.hc, n_embd, o0, o1, tid, kSThreads);
    // the last block to get here puts the slot counters back to zero for the next launch on this scratch
    if (tid == 0) {
        __threadfence();
        const unsigned done = atomicAdd(&G.ecnt[15], 1u);
        if (done == gridDim.x - 1u) {
            if (good) {
                for (int i = 0; i < kSlotsMax; ++i) G.ecnt[i] = 0u;
                G.ecnt[15] = 0u;
            }
            if (A.ar.nm >= 2 && A.ar_seq == 0u && A.ar.seq_counter != nullptr) *(volatile unsigned*) A.ar.seq_counter = sh.ar_seq;
            s_stamp(A.sync, 5);
            __threadfence();
        }
    }
}

template<int T, int TS>
int launch_stream(const FusedArgs& A, size_t smem, cudaStream_t s) {
    static std::atomic<int> attr_dev{-1};
    static std::atomic<size_t> attr_smem{0};
    static thread_local int cached_dev = -1, cached_grid = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (cached_dev != dev) {
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cached_grid = sms;
        cached_dev = dev;
    }
    if (attr_dev.load() != dev || attr_smem.load() < smem) {
        if (cudaFuncSetAttribute(moe_layer_t1_stream_kernel<T, TS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess)
            return note_launch("stream smem attribute");
        attr_dev.store(dev);
        attr_smem.store(smem);
    }
    const int grid = cached_grid;
    if (4 * ((A.n_embd / 4 + grid - 1) / grid) > kMaxRows) return refuse(MAYA_ERR_LIMIT);
    if (A.ar.nm >= 2 && grid > MAYA_PEER_AR_BLOCKS) return refuse(MAYA_ERR_LIMIT);
    FusedArgs args = A;
    void* params[] = {&args};
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kSThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 2;
    cudaLaunchKernelExC(&cfg, (const void*) moe_layer_t1_stream_kernel<T, TS>, params);
    return note_launch("moe_layer_t1_stream");
}

size_t stream_smem(const maya_moe_layer& L, int T) {
    const int h_ld = L.n_ff > L.n_ff_sh ? L.n_ff : L.n_ff_sh;
    const int slot = T == MAYA_IQ3_S ? Stage<MAYA_IQ3_S>::bytes : Stage<MAYA_IQ2_S>::bytes;
    const size_t tab = T == MAYA_IQ3_S ? (size_t) kRepTabBytes<MAYA_IQ3_S> : (size_t) kRepTabBytes<MAYA_IQ2_S>;
    return tab + ximg_bytes(L.n_embd / 32) + (size_t) kSlotsMax * ximg_bytes(h_ld / 32) + (size_t) kDotWarps * kSlots * slot +
           (size_t) L.n_expert * sizeof(double);
}

}  // namespace

// bytes of the layer scratch's h area this kernel needs
size_t stream_scratch_bytes(int h_ld) {
    const int nb = h_ld / 32;
    return (size_t) kSlotsMax * h_ld * 5 + (size_t) kSlotsMax * nb * 8 + 16 * sizeof(unsigned);
}

// Whether the streamed single-token kernel covers this layer (else the grid-barrier kernel or the staged kernels run).
bool stream_t1_supported(const maya_moe_layer& L) {
    if (L.gu_type != L.d_type || L.gu_type != MAYA_IQ2_S) return false;
    if (L.n_embd % Stage<MAYA_IQ2_S>::seg_vals || L.n_ff % Stage<MAYA_IQ2_S>::seg_vals) return false;
    if (L.n_embd / Stage<MAYA_IQ2_S>::seg_vals > 8 || L.n_ff / Stage<MAYA_IQ2_S>::seg_vals > 8) return false;
    if (L.n_ff_sh > 0 && L.shared_here) {
        if (L.sh_gu_type != MAYA_Q8_0 || L.sh_d_type != MAYA_Q8_0) return false;
        if (L.n_embd % Stage<MAYA_Q8_0>::seg_vals || L.n_ff_sh % Stage<MAYA_Q8_0>::seg_vals) return false;
        if (L.n_embd / Stage<MAYA_Q8_0>::seg_vals > 8 || L.n_ff_sh / Stage<MAYA_Q8_0>::seg_vals > 8) return false;
        if (L.sh_lo != 0 || (L.sh_hi != 0 && L.sh_hi != L.n_ff_sh)) return false;     // a width slice: the other kernel
    }
    if (L.n_expert > kRouteThreads * kRouterMaxPerThread) return false;
    if (L.n_embd % 4 || L.n_embd > (1 << 21)) return false;
    if (stream_smem(L, L.gu_type) > 227 * 1024 - sizeof(StreamShared) - 1024) return false;
    return true;
}

int stream_t1(const maya_moe_layer& L, const float* logits, const void* x, int x_is_bf16, int* ids, float* weights,
              float* out, float* h_scratch, unsigned* sync, const maya_peer_ar* ar, int ar_rank, unsigned ar_seq,
              const maya_hc_post_args* hc, cudaStream_t s) {
    FusedArgs A{};
    if (hc != nullptr) A.hc = *hc;
    if (ar != nullptr) { A.ar = *ar; A.ar_rank = ar_rank; A.ar_seq = ar_seq; }
    A.logits = logits; A.x = x; A.x_is_bf16 = x_is_bf16;
    A.n_embd = L.n_embd; A.n_ff = L.n_ff; A.n_expert = L.n_expert; A.k = L.k;
    A.experts = (const uint8_t*) L.experts; A.expert_stride = L.expert_stride;
    A.expert_lo = L.expert_lo; A.expert_hi = L.expert_hi;
    const bool sh = L.n_ff_sh > 0 && L.shared_here && L.shared != nullptr;
    A.shared = sh ? (const uint8_t*) L.shared : nullptr;
    A.n_ff_sh = sh ? L.n_ff_sh : 0;
    A.sh_lo = 0;
    A.sh_hi = A.n_ff_sh;
    A.limit = L.limit;
    A.ids = ids; A.weights = weights; A.out = out; A.h = h_scratch; A.sync = sync;
    const size_t smem = stream_smem(L, L.gu_type);
    return sh ? launch_stream<MAYA_IQ2_S, MAYA_Q8_0>(A, smem, s) : launch_stream<MAYA_IQ2_S, 0>(A, smem, s);
}

}  // namespace maya
