// moe_fused.cu - one token through one MoE layer in ONE persistent kernel: route, quantize the activation, routed and
// shared gate/up + SwiGLU, q8_1 of h, routed and shared down, weighted combine.
//
// The reference spends 3-6 launches a layer on this (Glm5Model::fast_moe, src/core/glm_fast_path.cu:6917-7100: router
// GEMV launch, moe_route, moe_gate_up, moe_down; native path: 4 launches inside native_expert_grouped alone).  At
// ~137 MB a token the whole layer is ~21 us of HBM time on a B200, so launch gaps and per-kernel tails would cost as
// much as the work.  Here one cooperative grid of one block per SM does it:
//
//   phase 0 (every block, redundantly - no grid-wide dependency): warps 0-7 route the token (the same bits in every
//            block); warps 8-31 build the replicated codebook in shared memory and quantize x to q8_1 there;
//   phase 1  a unit = 32 consecutive FFN rows of one expert (the shared expert's units follow the routed ones); block b
//            takes units b, b + grid, ...; a warp item is two FFN rows (their gate and up rows share the activation
//            registers); the block that computed a unit rounds its 32 h values to one q8_1 block and writes it to the
//            scratch;
//   grid barrier (a wait on a counter in the caller's scratch, bounded by %globaltimer; a time-out sets a sticky error
//            word, and every thread of the block then skips phase 2, the cross-rank exchange and the residual write);
//   phase 2  every block copies the q8_1 image of h ((k + 1) x n_ff / 32 blocks) to shared memory, then owns a
//            contiguous slice of the output rows: items are (row pair, expert); the per-expert partials meet in shared
//            memory and one thread per row runs the combine chain in plan order.
//
// Every (row, expert) dot, the q8_1 of h and the combine chain use the operations and order of the staged kernels
// (moe_decode.cu), so the output is bit-identical to maya_moe_gate_up + maya_moe_down on the same plan.
#include <cooperative_groups.h>

#include "maya_dots_t1.cuh"
#include "maya_internal.cuh"
#include "maya_peer_ar.cuh"
#include <atomic>
#include <type_traits>

#include "maya_hc_post.cuh"
#include "maya_router.cuh"
#include "maya_fused_args.cuh"

namespace maya {
namespace {

constexpr int kFusedThreads = 1024;
constexpr int kRouteThreads = 256;
constexpr int kMaxSliceRows = 96;          // output rows a block may own (n_embd / grid rounded up)
constexpr unsigned long long kBarrierTimeoutNs = 1000000000ull;   // the grid barrier gives up after a second


constexpr int kUnitBatch = 4;   // units of 32 FFN rows a block works on at a time (64 four-row items: two per warp)

struct FusedShared {
    RouterShared route;
    unsigned long long ptr[MAYA_MAX_K + 1];
    float w[MAYA_MAX_K];
    float part[kMaxSliceRows][MAYA_MAX_K + 1];
    unsigned epoch;
    unsigned ar_seq;
    int ve[MAYA_MAX_K];        // the plan entries this rank computes (blob address != 0), in plan order
    int nv;
    float hbuf[kUnitBatch][32];   // the h values of the (expert, 32-row group) units this block is working on
    int bar_ok;                   // the grid barrier's outcome, for every thread of the block
};

// balanced contiguous split of n rows over nb blocks
__device__ __forceinline__ void slice(int n, int nb, int b, int& r0, int& r1) {
    const int base = n / nb, rem = n % nb;
    r0 = b * base + min(b, rem);
    r1 = r0 + base + (b < rem ? 1 : 0);
}

// q8_1 of 32 values (one per lane) straight into the shared structure-of-arrays form the dots read.
__device__ __forceinline__ void q8_1_to_smem(float v, int4* q, float* d, int* isum, int blk, int lane) {
    const float amax = warp_max(fabsf(v));
    const float dd = fminf(__fdiv_rn(amax, 127.0f), 65504.0f);
    const int qi = amax == 0.0f ? 0 : (int) fmaxf(-127.0f, fminf(127.0f, roundf(__fdiv_rn(v, dd))));
    ((int8_t*) q)[blk * 32 + lane] = (int8_t) qi;
    int s = qi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) {
        d[blk] = __half2float(__float2half_rn(dd));   // the scale as the f16 block field holds it
        isum[blk] = s;
    }
}

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// block 0's wall-clock stamp of a phase boundary (a 64-bit ns count in two scratch words)
__device__ __forceinline__ void stamp(unsigned* sync, int i) {
    if (blockIdx.x == 0 && threadIdx.x == 0) *(volatile unsigned long long*) &sync[4 + 2 * i] = global_ns();
}

// All blocks of the (cooperative) grid meet here.  false in EVERY thread of the block when the wait ran out: thread 0
// leaves the outcome in shared memory before the closing barrier.
__device__ __forceinline__ bool grid_barrier(unsigned* sync, unsigned epoch, int* s_ok) {
    __syncthreads();
    if (threadIdx.x == 0) {
        int ok = 1;
        __threadfence();
        atomicAdd(&sync[0], 1u);
        const unsigned target = (epoch + 1u) * gridDim.x;
        const unsigned long long t0 = global_ns();
        while ((int) (*(volatile unsigned*) &sync[0] - target) < 0) {
            if (global_ns() - t0 > kBarrierTimeoutNs) { ok = 0; atomicExch(&sync[2], 1u); break; }
            __nanosleep(20);
        }
        __threadfence();
        *s_ok = ok;
    }
    __syncthreads();
    return *s_ok != 0;
}

// RT: the router - 0 softmax, 1 sigmoid.  A template parameter, not a branch on A.router: with both routers compiled into
// one kernel the softmax layer's routing phase ran 2 us longer (the 64-register cap of a 1024-thread block is shared by
// everything the phase may call).
// The token's routing by the block's first kRouteThreads threads, as a function of its own: run once a launch, it is
// kept out of the kernel's register allocation and instruction scheduling (which proved sensitive to what phase 0 holds).
template<int RT>
__device__ __noinline__ void route_token(const float* logits, const float* bias, int n_expert, int k, float w_scale, int norm_w,
                                         int tid, double* s_ex, RouterShared* route) {
    using RS = NamedSync<1, kRouteThreads>;
    const int per = (n_expert + kRouteThreads - 1) / kRouteThreads;
    if constexpr (RT == 1) {
        if (per <= 1) route_sigmoid<1, RS>(logits, bias, n_expert, k, w_scale, norm_w, tid, kRouteThreads, *route);
        else if (per <= 2) route_sigmoid<2, RS>(logits, bias, n_expert, k, w_scale, norm_w, tid, kRouteThreads, *route);
        else if (per <= 4) route_sigmoid<4, RS>(logits, bias, n_expert, k, w_scale, norm_w, tid, kRouteThreads, *route);
        else route_sigmoid<8, RS>(logits, bias, n_expert, k, w_scale, norm_w, tid, kRouteThreads, *route);
    } else {
        if (per <= 1) route_softmax<1, RS>(logits, n_expert, k, tid, kRouteThreads, s_ex, *route);
        else if (per <= 2) route_softmax<2, RS>(logits, n_expert, k, tid, kRouteThreads, s_ex, *route);
        else if (per <= 4) route_softmax<4, RS>(logits, n_expert, k, tid, kRouteThreads, s_ex, *route);
        else route_softmax<8, RS>(logits, n_expert, k, tid, kRouteThreads, s_ex, *route);
    }
}

// HV: the kernel may cut phase-1 units in halves (decided per launch on the device; the code for it is compiled in only
// where a rank's units can be that few - in the one-GPU kernel it cost 1 us by its mere presence).
template<int T, int TS, int RT, bool HV>
__global__ void __launch_bounds__(kFusedThreads, 1) moe_layer_t1_kernel(FusedArgs A) {
    extern __shared__ __align__(16) uint8_t s_raw[];
    __shared__ FusedShared sh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int NW = kFusedThreads / 32;
    const int k = A.k, n_embd = A.n_embd, n_ff = A.n_ff;
    const bool has_sh = TS != 0 && A.shared != nullptr;
    const int ne = k + (has_sh ? 1 : 0);             // experts incl. the shared one (index k)
    const int h_ld = max(n_ff, A.n_ff_sh);

    // shared-memory carve-up: [replicated codebook | activation columns (x, later the h of every expert) | exp scratch]
    uint32_t* s_tab = (uint32_t*) s_raw;
    uint8_t* s_cols = s_raw + kRepTabBytes<T>;
    const int nblk_x = n_embd / 32, nblk_h = h_ld / 32;
    const int cols_blocks = (max(nblk_x, (MAYA_MAX_K + 1) * nblk_h) + 1) & ~1;   // even: the router's scratch is 16-byte aligned
    int4* cq = (int4*) s_cols;
    float* cd = (float*) (s_cols + (size_t) cols_blocks * 32);
    int* cs = (int*) (s_cols + (size_t) cols_blocks * 36);
    double* s_ex = (double*) (s_cols + (size_t) cols_blocks * 40);

    // Programmatic dependent launch: the next launch on the stream may be set up while this one runs, and this one may
    // have started before the launch in front of it ended.  Nothing of global memory is read or written before
    // grid_dependency_wait() (only the codebook, a constant of the library, is copied to shared memory before it ...);
    // without the launch attribute both instructions do nothing.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // ... and the token's logits and activations are asked into L2 (a prefetch reads nothing into the SM: whatever the
    // launch in front still writes there is read after the wait, from L2, the point of coherence)
    if (tid < kRouteThreads) {
        if (tid * 32 < A.n_expert) asm volatile("prefetch.global.L2 [%0];" ::"l"(A.logits + tid * 32));
    } else {
        const int t2 = tid - kRouteThreads;
        const size_t xb = (size_t) n_embd * (A.x_is_bf16 ? 2 : 4);
        if ((size_t) t2 * 128 < xb) asm volatile("prefetch.global.L2 [%0];" ::"l"((const uint8_t*) A.x + (size_t) t2 * 128));
        load_tab_rep<T>(s_tab, t2, kFusedThreads - kRouteThreads);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) {
        sh.epoch = *(volatile unsigned*) &A.sync[1];
        sh.ar_seq = ar_seq_begin(A.ar, A.ar_seq);
    }
    stamp(A.sync, 0);

    // ---------------------------------------------------------------- phase 0
    if (tid < kRouteThreads) {
        route_token<RT>(A.logits, A.router_bias, A.n_expert, k, A.router_w_scale, A.router_norm_w, tid, s_ex, &sh.route);
        if (tid < k) {
            const int e = sh.route.ids[tid];
            sh.w[tid] = sh.route.val[tid];
            sh.ptr[tid] = (e >= A.expert_lo && e < A.expert_hi)
                              ? (unsigned long long) (A.experts + (size_t) e * A.expert_stride) : 0ull;
            if (blockIdx.x == 0) { A.ids[tid] = e; A.weights[tid] = sh.route.val[tid]; }
        }
        if (tid == 0) sh.ptr[k] = has_sh ? (unsigned long long) A.shared : 0ull;
        NamedSync<1, kRouteThreads>::sync();
        if (tid == 0) {     // compact the entries that are this rank's: skipped ones must not leave warps idle
            int nv = 0;
            for (int i = 0; i < k; ++i)
                if (sh.ptr[i] != 0ull) sh.ve[nv++] = i;
            sh.nv = nv;
        }
    } else {
        const int t2 = tid - kRouteThreads;
        // the token's activations: 8 loads in flight per lane before the first is used (they come from HBM)
        constexpr int NW2 = (kFusedThreads - kRouteThreads) / 32;
        for (int b0 = (t2 >> 5); b0 < nblk_x; b0 += 8 * NW2) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int b = b0 + i * NW2;
                v[i] = 0.0f;
                if (b < nblk_x)
                    v[i] = A.x_is_bf16 ? __uint_as_float((uint32_t) ((const uint16_t*) A.x)[b * 32 + lane] << 16)
                                       : ((const float*) A.x)[b * 32 + lane];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (b0 + i * NW2 < nblk_x) q8_1_to_smem(v[i], cq, cd, cs, b0 + i * NW2, lane);
        }
    }
    __syncthreads();
    stamp(A.sync, 1);
    XCols X;
    X.q = cq; X.d = cd; X.isum = cs; X.nblk = nblk_x;

    // ---------------------------------------------------------------- phase 1: gate / up + SwiGLU + q8_1(h)
    // A unit = 32 consecutive FFN rows of one expert = one q8_1 block of its h; block b takes units b, b + grid, ...
    // The block that computed a unit also rounds it to q8_1 and writes the block to the scratch, so that after the grid
    // barrier every block only COPIES the (k + 1) x n_ff / 32 blocks into shared memory (23 KB on the benchmark layer)
    // instead of all 148 reading the same f32 h and rounding it again (that cost 12 us of L2 contention and arithmetic).
    // The q8_1 image in the scratch: [unit][32] int8, then [unit] f32 scales, then [unit] int sums (unit = e * nblk_h + g).
    int8_t* const gq = (int8_t*) A.h;
    float* const gd = (float*) (gq + (size_t) ne * nblk_h * 32);
    int* const gs = (int*) (gd + (size_t) ne * nblk_h);
    {
        const int ng = n_ff / 32, units_r = sh.nv * ng, ng_sh = has_sh ? (A.sh_hi - A.sh_lo) / 32 : 0, U = units_r + ng_sh;
        const size_t rb = row_bytes(T, n_embd);
        // Unit SLOTS are handed to the blocks in order; which unit sits in a slot spreads the shared expert's units
        // evenly among the routed ones (slot s holds a shared unit where floor(s * ng_sh / U) steps).  Numbered after
        // the routed units they all fell into the blocks' last round, 27 MB of Q8_0 rows wanted at once by 64 SMs - an
        // HBM-bound tail behind an issue-bound phase.  Below, u is a unit in the old numbering: routed [0, units_r), shared after.
        // (Only with more than two rounds of units a block: with two or fewer - a width slice at 2 or more GPUs - the
        // spread measured slower, 43.4 against 40.7 us on the half-width slice.)
        const bool spread = !HV && ng_sh > 0 && U > 2 * (int) gridDim.x;    // (HV kernels serve ranks with few units)
        auto unit_of = [&](int slot) -> int {
            if (!spread) return slot;
            const int c0 = slot * ng_sh / U, c1 = (slot + 1) * ng_sh / U;
            return c1 > c0 ? units_r + c0 : slot - c0;
        };
        // Fewer units than half the grid (a rank's share at 8 GPUs): a unit is cut into two halves of 16 FFN rows for two
        // blocks - one weight row a warp - so that twice as many SMs pull rows.  A half leaves its 16 h values as f32 in
        // the scratch; the block that brings the unit's counter to an odd value found the other half there already and
        // rounds the 32 values to the unit's q8_1 block (the same 32 values, the same rounding: the same bits).
        const bool halves = HV && U > 0 && 2 * U <= (int) gridDim.x;
        if (HV && halves) {
            float* const hst = (float*) ((uint8_t*) A.h + (size_t) (MAYA_MAX_K + 1) * nblk_h * 40);
            unsigned* const hcnt = (unsigned*) (hst + (size_t) (MAYA_MAX_K + 1) * nblk_h * 32);
            if ((int) blockIdx.x < 2 * U) {
                const int u = unit_of((int) blockIdx.x >> 1), half = (int) blockIdx.x & 1;
                const int fr = 16 * half + (warp >> 1), mat = warp & 1;         // FFN row in the unit; gate (0) or up (1)
                int e, g;
                float o[1] = {0.0f};
                if (u < units_r) {
                    const int ei = u / ng;
                    e = sh.ve[ei];
                    g = u - ei * ng;
                    const uint8_t* rows[1] = {(const uint8_t*) sh.ptr[e] + (size_t) (mat * n_ff + g * 32 + fr) * rb};
                    rows_dot1<T, 1>(rows, X, n_embd, lane, s_tab, o);
                } else {
                    e = k;
                    g = A.sh_lo / 32 + (u - units_r);
                    if constexpr (TS != 0) {
                        const uint8_t* rows[1] = {A.shared + (size_t) (mat * A.n_ff_sh + g * 32 + fr) * row_bytes(TS, n_embd)};
                        rows_dot1<TS, 1>(rows, X, n_embd, lane, nullptr, o);
                    }
                }
                if (lane == 0) sh.hbuf[0][warp] = o[0];
                __syncthreads();
                if (warp == 0) {
                    const int slot = e * nblk_h + g;
                    if (lane < 16) __stcg(&hst[(size_t) slot * 32 + 16 * half + lane], swiglu(sh.hbuf[0][2 * lane], sh.hbuf[0][2 * lane + 1], A.limit));
                    __threadfence();
                    __syncwarp();
                    unsigned old = 0u;
                    if (lane == 0) old = atomicAdd(&hcnt[slot], 1u);
                    old = __shfl_sync(0xffffffffu, old, 0);
                    if (old & 1u) {                                              // the other half is in place
                        __threadfence();
                        q8_1_to_smem(__ldcg(&hst[(size_t) slot * 32 + lane]), (int4*) gq, gd, gs, slot, lane);
                    }
                }
            }
        } else
        for (int u0 = blockIdx.x; u0 < U; u0 += gridDim.x * kUnitBatch) {
            int nu = 0;                                          // units of this batch: u0, u0 + grid, ...
            for (int u = u0; u < U && nu < kUnitBatch; u += gridDim.x) ++nu;
            // an item = two FFN rows of a unit: their gate rows and up rows, four weight rows sharing the activation
            // registers (more field loads in flight per warp than one row pair).  An odd last unit would leave half the
            // warps idle for a whole item: it is done one FFN row a warp instead (all 32 busy for half as long) - what a
            // rank with few experts mostly has.
            static_assert(NW == 32, "a unit's 32 FFN rows map onto the block's 32 warps");
            const int nu4 = nu & ~1;
            for (int it = warp; it < nu4 * 16; it += NW) {
                const int j = it >> 4, u = unit_of(u0 + j * (int) gridDim.x), ra_in = 2 * (it & 15);
                float o[4];
                if (u < units_r) {
                    const int ei = u / ng, ra = (u - ei * ng) * 32 + ra_in, e = sh.ve[ei];
                    const uint8_t* blob = (const uint8_t*) sh.ptr[e];
                    const uint8_t* rows[4] = {blob + (size_t) ra * rb, blob + (size_t) (n_ff + ra) * rb,
                                              blob + (size_t) (ra + 1) * rb, blob + (size_t) (n_ff + ra + 1) * rb};
                    rows_dot1<T, 4>(rows, X, n_embd, lane, s_tab, o);
                } else if constexpr (TS != 0) {
                    const int ra = A.sh_lo + (u - units_r) * 32 + ra_in;
                    const size_t rbs = row_bytes(TS, n_embd);
                    const uint8_t* rows[4] = {A.shared + (size_t) ra * rbs, A.shared + (size_t) (A.n_ff_sh + ra) * rbs,
                                              A.shared + (size_t) (ra + 1) * rbs, A.shared + (size_t) (A.n_ff_sh + ra + 1) * rbs};
                    rows_dot1<TS, 4>(rows, X, n_embd, lane, nullptr, o);
                }
                if (lane == 0) {
                    sh.hbuf[j][ra_in] = swiglu(o[0], o[1], A.limit);
                    sh.hbuf[j][ra_in + 1] = swiglu(o[2], o[3], A.limit);
                }
            }
            if (nu & 1) {
                const int u = unit_of(u0 + nu4 * (int) gridDim.x);
                float o[2];
                if (u < units_r) {
                    const int ei = u / ng, ra = (u - ei * ng) * 32 + warp, e = sh.ve[ei];
                    const uint8_t* blob = (const uint8_t*) sh.ptr[e];
                    const uint8_t* rows[2] = {blob + (size_t) ra * rb, blob + (size_t) (n_ff + ra) * rb};
                    rows_dot1<T, 2>(rows, X, n_embd, lane, s_tab, o);
                } else if constexpr (TS != 0) {
                    const int ra = A.sh_lo + (u - units_r) * 32 + warp;
                    const size_t rbs = row_bytes(TS, n_embd);
                    const uint8_t* rows[2] = {A.shared + (size_t) ra * rbs, A.shared + (size_t) (A.n_ff_sh + ra) * rbs};
                    rows_dot1<TS, 2>(rows, X, n_embd, lane, nullptr, o);
                }
                if (lane == 0) sh.hbuf[nu4][warp] = swiglu(o[0], o[1], A.limit);
            }
            __syncthreads();
            if (warp < nu) {                                     // one warp rounds one unit
                const int u = unit_of(u0 + warp * (int) gridDim.x);
                int e, g;
                if (u < units_r) { const int ei = u / ng; e = sh.ve[ei]; g = u - ei * ng; }
                else { e = k; g = A.sh_lo / 32 + (u - units_r); }
                q8_1_to_smem(sh.hbuf[warp][lane], (int4*) gq, gd, gs, e * nblk_h + g, lane);
            }
            __syncthreads();
        }
    }
    // Output rows of this block.  With a cross-rank sum in the epilogue the slice is whole float4s (it moves 16 bytes a
    // lane); without one, whole row pairs: with 6144 rows over 148 blocks that is 20-21 pairs a block instead of 10-11
    // quads, i.e. at most 189 (pair, expert) items = 6 rounds of the 32 warps where 44 rows would need a 7th for 6 items.
    int o0, o1;
    const int gran = A.ar.nm >= 2 ? 4 : 2;
    slice(n_embd / gran, gridDim.x, blockIdx.x, o0, o1);
    o0 *= gran;
    o1 *= gran;
    const int nrows = o1 - o0;
    const size_t drb = row_bytes(T, n_ff), down_off = 2 * (size_t) n_ff * row_bytes(T, n_embd);
    // A phase-2 item = a few of this block's output rows against one expert's h.  Rows of 64 or more calls (2048
    // values of an i-quant): two rows, all lanes on each.  Shorter rows - a width slice of an expert - are taken four
    // at a time per lane group, and 32 / calls lane groups side by side when a row has fewer than 32 calls, so that an
    // item keeps every lane busy and a block needs 1-3 rounds of its warps instead of 6 ever shorter ones.
    struct DownShape { int calls, groups, rpi, items; };
    auto shape = [&](int calls) {
        DownShape d;
        d.calls = calls;
        d.groups = (calls < 32 && (calls & (calls - 1)) == 0) ? 32 / calls : 1;
        d.rpi = (calls <= 32 ? 4 : 2) * d.groups;
        d.items = (nrows + d.rpi - 1) / d.rpi;
        return d;
    };
    const DownShape dr = shape(calls_per_row<T>(n_ff));
    DownShape ds = dr;
    if constexpr (TS != 0) ds = shape(calls_per_row<TS>(has_sh ? A.sh_hi - A.sh_lo : n_ff));
    __syncthreads();
    stamp(A.sync, 2);
    const bool ok = grid_barrier(A.sync, sh.epoch, &sh.bar_ok);
    stamp(A.sync, 3);

    // ---------------------------------------------------------------- phase 2: q8_1(h), down, combine
    if (ok) {
        // every block needs all of q8_1(h): a plain copy of what the producers wrote (through L2: other SMs wrote it)
        {
            const int nb = ne * nblk_h;
            const uint4* src = (const uint4*) gq;
            uint4* dst = (uint4*) cq;
            for (int i = tid; i < nb * 2; i += kFusedThreads) dst[i] = __ldcg(src + i);
            for (int i = tid; i < nb; i += kFusedThreads) { cd[i] = __ldcg(gd + i); cs[i] = __ldcg(gs + i); }
        }
        __syncthreads();
        // One loop per (expert class, item shape), chosen outside it: a single loop that branched per item between the
        // shapes cost the common case 2.6 us.  The item index runs on from the routed class into the shared one, so the
        // warps stay evenly loaded.
        const int items_r = sh.nv * dr.items, items_all = items_r + (has_sh ? ds.items : 0);
        const int n_sh_first = HV ? items_all - items_r : 0, n_r_first = HV ? 0 : items_r;   // items of the class that goes first
        auto run = [&](auto type_c, auto nr_c, auto short_c, auto routed_c, int it, int it_end, const DownShape& d) {
            constexpr int TY = decltype(type_c)::value, NR = decltype(nr_c)::value;
            constexpr bool SHORT = decltype(short_c)::value, ROUTED = decltype(routed_c)::value;
            for (; it < it_end; it += NW) {
                const int li = ROUTED ? it - n_sh_first : it - n_r_first;
                const int ei = ROUTED ? li / d.items : 0, grp = li - ei * d.items;
                const int e = ROUTED ? sh.ve[ei] : k;
                const int r0 = grp * d.rpi + (SHORT ? lane / d.calls : 0);      // this lane's first row; then + groups
                XCols H;
                H.q = cq + (size_t) 2 * e * nblk_h; H.d = cd + (size_t) e * nblk_h; H.isum = cs + (size_t) e * nblk_h;
                H.nblk = nblk_h;
                const uint8_t* base;
                size_t pitch;
                int n_in;
                if constexpr (ROUTED) {
                    base = (const uint8_t*) sh.ptr[e] + down_off;
                    pitch = drb;
                    n_in = n_ff;
                } else {                             // this rank's columns [sh_lo, sh_hi) of the shared expert's down rows
                    const int b0 = A.sh_lo / 32;
                    pitch = row_bytes(TY, A.n_ff_sh);
                    base = A.shared + 2 * (size_t) A.n_ff_sh * row_bytes(TY, n_embd) + row_bytes(TY, A.sh_lo);
                    n_in = A.sh_hi - A.sh_lo;
                    H.q += 2 * b0; H.d += b0; H.isum += b0; H.nblk = n_in / 32;
                }
                const uint8_t* rows[NR];
#pragma unroll
                for (int r = 0; r < NR; ++r) rows[r] = base + (size_t) (o0 + min(r0 + r * d.groups, nrows - 1)) * pitch;
                float o[NR];
                const uint32_t* tab = ROUTED ? s_tab : nullptr;
                if constexpr (SHORT) rows_dot1_short<TY, NR>(rows, H, d.calls, lane, tab, o);
                else rows_dot1<TY, NR>(rows, H, n_in, lane, tab, o);
                if (SHORT ? (lane & (d.calls - 1)) == 0 : lane == 0) {
#pragma unroll
                    for (int r = 0; r < NR; ++r)
                        if (r0 + r * d.groups < nrows) sh.part[r0 + r * d.groups][e] = o[r];
                }
            }
            return it;
        };
        using std::integral_constant;
        using std::true_type;
        using std::false_type;
        int it = warp;
        auto run_shared = [&](int it0, int it1) -> int {
            if constexpr (TS != 0) {
                if (!has_sh) return it0;
                if (ds.groups > 1) return run(integral_constant<int, TS>{}, integral_constant<int, 4>{}, true_type{}, false_type{}, it0, it1, ds);
                if (ds.rpi == 4) return run(integral_constant<int, TS>{}, integral_constant<int, 4>{}, false_type{}, false_type{}, it0, it1, ds);
                return run(integral_constant<int, TS>{}, integral_constant<int, 2>{}, false_type{}, false_type{}, it0, it1, ds);
            } else {
                return it0;
            }
        };
        auto run_routed = [&](int it0, int it1) -> int {
            if (dr.groups > 1) return run(integral_constant<int, T>{}, integral_constant<int, 4>{}, true_type{}, true_type{}, it0, it1, dr);
            if (dr.rpi == 4) return run(integral_constant<int, T>{}, integral_constant<int, 4>{}, false_type{}, true_type{}, it0, it1, dr);
            return run(integral_constant<int, T>{}, integral_constant<int, 2>{}, false_type{}, true_type{}, it0, it1, dr);
        };
        // which class goes first is the kernel variant's: measured, the shared expert's rows first suit a rank's slice
        // (half-width slice 40.9 -> 39.4 us) and last suit the whole layer (59.9 against 60.5 us)
        if constexpr (HV) { it = run_shared(it, n_sh_first); run_routed(it, items_all); }
        else { it = run_routed(it, items_r); run_shared(it, items_all); }
        __syncthreads();
        if (tid < nrows) {
            float m = 0.0f;
            for (int i = 0; i < k; ++i) m = __fmaf_rn(sh.w[i], sh.ptr[i] != 0ull ? sh.part[tid][i] : 0.0f, m);
            if (A.cpu_flag != nullptr && *A.cpu_flag) m = __fadd_rn(m, A.cpu_part[o0 + tid]);    // the host lane's answer (moe_down's order)
            A.out[o0 + tid] = __fadd_rn(m, has_sh ? sh.part[tid][k] : 0.0f);
        }
    }
    stamp(A.sync, 4);
    // ---------------------------------------------------------------- epilogue: the cross-rank sum of this block's rows
    // After a barrier time-out `out` was not computed: nothing is sent (the peers' waits run out into their own sticky
    // error) and the residual is not written.  After a failed exchange `out` is undefined: no residual write either.
    bool final_ok = ok;
    if (A.ar.nm >= 2) {
        __syncthreads();
        int u0, u1;
        slice(n_embd / 4, gridDim.x, blockIdx.x, u0, u1);
        if (ok) final_ok = peer_allreduce_block_words(A.out, u0, u1, A.ar, A.ar_rank, sh.ar_seq, blockIdx.x);
        else if (tid == 0) atomicOr(A.ar.error, 1u);
    }
    __syncthreads();
    if (A.hc.R_new != nullptr && final_ok) {    // the consumer of `out`: this block's rows are final (and the same on every rank)
        int e0 = o0, e1 = o1;
        if (A.ar.nm >= 2) { slice(n_embd / 4, gridDim.x, blockIdx.x, e0, e1); e0 *= 4; e1 *= 4; }
        hc_post_rows(A.out, A.hc, n_embd, e0, e1, tid, kFusedThreads);
    }
    stamp(A.sync, 5);
    // the launch's last word: the next launch on this scratch (stream-ordered) starts a new epoch
    if (blockIdx.x == 0 && tid == 0) {
        *(volatile unsigned*) &A.sync[1] = sh.epoch + 1u;
        if (A.ar.nm >= 2 && A.ar_seq == 0u && A.ar.seq_counter != nullptr) *(volatile unsigned*) A.ar.seq_counter = sh.ar_seq;
    }
}

template<int T, int TS, int RT, bool HV>
int launch_fused_rt(const FusedArgs& A, cudaStream_t s) {
    // per instantiation: the device and dynamic shared-memory size the attribute was last set for, and whether the
    // programmatic-serialization attribute is in use (1), was refused by the driver (0) or has not been tried (-1)
    static std::atomic<int> attr_dev{-1}, pdl{-1};
    static std::atomic<size_t> attr_smem{0};
    static thread_local int cached_dev = -1, cached_grid = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    const int nblk_x = A.n_embd / 32, nblk_h = (A.n_ff > A.n_ff_sh ? A.n_ff : A.n_ff_sh) / 32;
    const int cols_blocks = ((nblk_x > (MAYA_MAX_K + 1) * nblk_h ? nblk_x : (MAYA_MAX_K + 1) * nblk_h) + 1) & ~1;
    const size_t smem = (size_t) kRepTabBytes<T> + (size_t) cols_blocks * 40 + (size_t) A.n_expert * sizeof(double);
    if (smem > 220 * 1024) return refuse(MAYA_ERR_LIMIT);
    if (cached_dev != dev) {
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cached_grid = sms;
        cached_dev = dev;
    }
    if (attr_dev.load() != dev || attr_smem.load() != smem) {
        if (cudaFuncSetAttribute(moe_layer_t1_kernel<T, TS, RT, HV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess)
            return note_launch("fused smem attribute");
        attr_dev.store(dev);
        attr_smem.store(smem);
    }
    int grid = cached_grid;
    if (4 * ((A.n_embd / 4 + grid - 1) / grid) > kMaxSliceRows || A.n_embd % 4) return refuse(MAYA_ERR_LIMIT);
    if (A.ar.nm >= 2 && grid > MAYA_PEER_AR_BLOCKS) return refuse(MAYA_ERR_LIMIT);
    FusedArgs args = A;
    void* params[] = {&args};
    // Cooperative (the grid barrier needs every block resident) and, where the driver accepts the attribute,
    // programmatically serialized after the launch in front of it: its set-up then overlaps that launch's tail.
    if (pdl.load() != 0) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(kFusedThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute at[2];
        at[0].id = cudaLaunchAttributeCooperative;
        at[0].val.cooperative = 1;
        at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = 2;
        const cudaError_t e = cudaLaunchKernelExC(&cfg, (const void*) moe_layer_t1_kernel<T, TS, RT, HV>, params);
        if (e == cudaSuccess) { pdl.store(1); return note_launch("moe_layer_t1"); }
        // only "this attribute / combination is not supported" turns the attribute off; any other failure is the launch's
        if (e != cudaErrorNotSupported && e != cudaErrorInvalidValue) return note_launch("moe_layer_t1");
        cudaGetLastError();
        pdl.store(0);
    }
    cudaLaunchCooperativeKernel((const void*) moe_layer_t1_kernel<T, TS, RT, HV>, dim3(grid), dim3(kFusedThreads), params, smem, s);
    return note_launch("moe_layer_t1");
}

template<int T, int TS>
int launch_fused(const FusedArgs& A, cudaStream_t s) {
    if (A.router == 1) return launch_fused_rt<T, TS, 1, false>(A, s);
    // units of one routed expert + the shared expert's: when even twice that many fit the grid, a rank with few local
    // experts (or a narrow width slice) may have fewer units than half the blocks
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    static thread_local int c_dev = -1, c_sms = 0;
    if (c_dev != dev) { cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); c_dev = dev; c_sms = sms; }
    const int units_min = A.n_ff / 32 + (A.shared != nullptr ? (A.sh_hi - A.sh_lo) / 32 : 0);
    return 2 * units_min <= c_sms ? launch_fused_rt<T, TS, 0, true>(A, s) : launch_fused_rt<T, TS, 0, false>(A, s);
}

}  // namespace

// Whether the fused single-token kernel covers this layer (else the staged kernels run).
bool fused_t1_supported(const maya_moe_layer& L) {
    if (L.gu_type != L.d_type || !type_is_core(L.gu_type)) return false;
    if (L.n_ff_sh > 0 && (L.sh_gu_type != MAYA_Q8_0 || L.sh_d_type != MAYA_Q8_0)) return false;
    if (L.n_expert > kRouteThreads * kRouterMaxPerThread) return false;
    return true;
}

int fused_t1(const maya_moe_layer& L, const float* logits, const void* x, int x_is_bf16, int* ids, float* weights,
             float* out, float* h_scratch, unsigned* sync, const maya_peer_ar* ar, int ar_rank, unsigned ar_seq,
             const maya_hc_post_args* hc, cudaStream_t s) {
    FusedArgs A{};
    if (hc != nullptr) A.hc = *hc;
    if (ar != nullptr) { A.ar = *ar; A.ar_rank = ar_rank; A.ar_seq = ar_seq; }
    A.logits = logits; A.x = x; A.x_is_bf16 = x_is_bf16;
    A.router = L.router; A.router_bias = L.router_bias; A.router_w_scale = L.router_w_scale; A.router_norm_w = L.router_norm_w;
    A.cpu_part = L.cpu_flag != nullptr ? L.cpu_part : nullptr; A.cpu_flag = L.cpu_flag;
    A.n_embd = L.n_embd; A.n_ff = L.n_ff; A.n_expert = L.n_expert; A.k = L.k;
    A.experts = (const uint8_t*) L.experts; A.expert_stride = L.expert_stride;
    A.expert_lo = L.expert_lo; A.expert_hi = L.expert_hi;
    const bool sh = L.n_ff_sh > 0 && L.shared_here && L.shared != nullptr && !(L.sh_hi > 0 && L.sh_hi <= L.sh_lo);
    A.shared = sh ? (const uint8_t*) L.shared : nullptr;
    A.n_ff_sh = sh ? L.n_ff_sh : 0;
    A.sh_lo = sh ? L.sh_lo : 0;
    A.sh_hi = sh ? (L.sh_hi > 0 ? L.sh_hi : L.n_ff_sh) : 0;
    A.limit = L.limit;
    A.ids = ids; A.weights = weights; A.out = out; A.h = h_scratch; A.sync = sync;
#define FUSED_CASE(TT)                                                      \
    case TT: return sh ? launch_fused<TT, MAYA_Q8_0>(A, s) : launch_fused<TT, 0>(A, s);
    switch (L.gu_type) {
        FUSED_CASE(MAYA_Q8_0)
        FUSED_CASE(MAYA_Q4_K)
        FUSED_CASE(MAYA_IQ2_S)
        FUSED_CASE(MAYA_IQ3_S)
        default: return refuse(MAYA_ERR_TYPE);
    }
#undef FUSED_CASE
}

}  // namespace maya
