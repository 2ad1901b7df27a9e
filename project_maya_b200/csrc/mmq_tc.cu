// mmq_tc.cu - the prompt path's grouped-by-expert GEMM over quantized expert matrices on the 5th-generation tensor
// cores: for every expert e, the activation rows [bounds[e], bounds[e+1]) times its [w_rows, w_cols] quantized matrix.
//
// Replaces mmq::quantize / mmq::Context::run / run_glu (include/strata/prefill/moe_mmq.hpp:59-99, src/prefill/
// moe_mmq.cu:114-228), which wrap llama.cpp's int8 `mma.sync` MMQ kernels (not part of the reference tree).  The
// reference rounds activations to q8_1 and multiplies integers with per-32 scales; an integer tcgen05 contraction
// would have to leave tensor memory every 32 values of K to apply those scales, so here both operands are expanded to
// f16 in shared memory - weights dequantized exactly as the format defines (f32, rounded once to f16), activations as
// d * q of their q8_1 image (the reference's rounding of x, kept so that results stay within its tolerance) - and
// multiplied by `tcgen05.mma.kind::f16` with f32 accumulators in tensor memory.
//
// One block = one 128-row slab of the weight matrix (gate and up slabs together for the fused SwiGLU form) x up to 128
// activation rows of one expert.  K advances 64 values a step through a 3-stage ring of shared-memory tiles: all 256
// threads dequantize a stage, one thread issues the four K = 16 MMAs of the stage and commits them to the stage's
// mbarrier, and the threads go on to the next stage while the tensor core works.  The epilogue reads the accumulators
// with tcgen05.ld (lane = weight row, column = activation row), applies SwiGLU for the fused form and writes
// dst[row][weight row] so that a warp stores 32 consecutive floats.
//
// Which expert and which of its 128-row groups a block handles is found on the device from `bounds` (a scan in shared
// memory), so no count ever travels to the host; the launch only needs an upper bound of the number of groups.
// Every mbarrier wait is bounded; a wait that runs out sets the error word and the block frees its tensor memory and
// returns.
#include <cuda_fp16.h>

#include <cstdio>

#include "maya_internal.cuh"
#include "maya_tcgen05.cuh"

namespace maya {
namespace {

constexpr int BM = 128, BN = 128, BK = 64, kStages = 3, kMmqThreads = 256;
constexpr int kTileBytes = BM * BK * 2;     // 16 KB: one operand tile of f16

__device__ __forceinline__ uint4 pack8(const float* v) {
    __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
    __half2 c = __floats2half2_rn(v[4], v[5]), d = __floats2half2_rn(v[6], v[7]);
    uint4 r;
    r.x = *(uint32_t*) &a; r.y = *(uint32_t*) &b; r.z = *(uint32_t*) &c; r.w = *(uint32_t*) &d;
    return r;
}
// 32 consecutive K-values of one row into the tile: chunks c0 .. c0 + 3
__device__ __forceinline__ void store32(uint8_t* tile, int rows, int r, int c0, const float* v) {
#pragma unroll
    for (int c = 0; c < 4; ++c) *(uint4*) (tile + (size_t) (c0 + c) * rows * 16 + r * 16) = pack8(v + 8 * c);
}

// weights of row `row`, K-tile kt (64 values), half h (32 values) -> f32
template<int T>
__device__ __forceinline__ void dequant32(const uint8_t* row, int kt, int h, float* v) {
    if constexpr (T == MAYA_Q4_K) {
        const uint8_t* blk = row + (size_t) (kt >> 2) * 144;
        const int j = kt & 3, sb = 2 * j + h;
        const uint32_t dm = ld_u32(blk);
        const float d = __half2float(__ushort_as_half((uint16_t) (dm & 0xFFFF)));
        const float dmin = __half2float(__ushort_as_half((uint16_t) (dm >> 16)));
        const uint8_t* s12 = blk + 4;
        int sc, mn;
        if (sb < 4) { sc = s12[sb] & 63; mn = s12[sb + 4] & 63; }
        else { sc = (s12[sb + 4] & 0x0F) | ((s12[sb - 4] >> 6) << 4); mn = (s12[sb + 4] >> 4) | ((s12[sb] >> 6) << 4); }
        const float dl = d * (float) sc, ml = dmin * (float) mn;
        const uint4 q0 = *(const uint4*) (blk + 16 + 32 * j), q1 = *(const uint4*) (blk + 32 + 32 * j);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t x = h ? (w[i] >> 4) : w[i];
#pragma unroll
            for (int b = 0; b < 4; ++b) v[4 * i + b] = dl * (float) ((x >> (8 * b)) & 0x0F) - ml;
        }
    } else {   // Q8_0
        const uint8_t* blk = row + (size_t) (2 * kt + h) * 34;
        const float d = ld_f16(blk);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t x = ld_u16(blk + 2 + 2 * i);
            v[2 * i] = d * (float) (int8_t) (x & 0xFF);
            v[2 * i + 1] = d * (float) (int8_t) (x >> 8);
        }
    }
}

// activation row (q8_1 blocks), K-tile kt, half h -> f32 values d * q
__device__ __forceinline__ void act32(const uint8_t* xrow, int kt, int h, float* v) {
    const uint8_t* b = xrow + (size_t) (2 * kt + h) * kQ81Bytes;
    const float d = ld_f16(b);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t x = ld_u32(b + 4 + 4 * i);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[4 * i + j] = d * (float) (int8_t) ((x >> (8 * j)) & 0xFF);
    }
}

struct MmqArgs {
    const uint8_t* w;
    size_t expert_bytes;
    int w_rows, w_cols;          // rows of one output (n_ff for the fused form: gate rows, then up rows), K
    int n;                       // experts of this product
    const int* expert_map;       // optional: expert i of the product is entry expert_map[i] of bounds
    const uint8_t* xq;           // q8_1 rows, w_cols / 32 blocks each
    const int* bounds;
    const int* ids;              // optional dst row of a sorted row
    float* dst;
    int64_t ld_dst;
    float limit;
    unsigned* error;             // optional sticky error word
};

template<int T, bool GLU>
__global__ void __launch_bounds__(kMmqThreads, 1) mmq_kernel(MmqArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_scan[kMmqThreads];
    __shared__ uint64_t s_done[kStages];
    __shared__ uint64_t s_final;
    __shared__ uint32_t s_tmem;
    __shared__ int s_fail;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- which (expert, 128-row group) is blockIdx.y: inclusive scan of the per-expert group counts
    //      (256 experts at a time; `base` carries the groups of the experts before the current 256)
    int found_e = -1, found_g = 0;
    {
        int base = 0;
        for (int e0 = 0; e0 < A.n && found_e < 0; e0 += kMmqThreads) {
            const int e = e0 + tid;
            int cnt = 0;
            if (e < A.n) {
                const int be = A.expert_map ? A.expert_map[e] : e;
                cnt = (A.bounds[be + 1] - A.bounds[be] + BN - 1) / BN;
            }
            s_scan[tid] = cnt;
            __syncthreads();
            for (int o = 1; o < kMmqThreads; o <<= 1) {
                const int v = tid >= o ? s_scan[tid - o] : 0;
                __syncthreads();
                s_scan[tid] += v;
                __syncthreads();
            }
            const int total = s_scan[kMmqThreads - 1];
            const int want = (int) blockIdx.y - base;
            if (want < total) {
                int lo = 0, hi = kMmqThreads - 1;       // the first entry whose inclusive sum exceeds `want`
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (s_scan[mid] > want) hi = mid; else lo = mid + 1;
                }
                found_e = e0 + lo;
                found_g = want - (lo > 0 ? s_scan[lo - 1] : 0);
            }
            base += total;
            __syncthreads();
        }
    }
    if (found_e < 0) return;                        // beyond the last group: uniform for the whole block
    const int be = A.expert_map ? A.expert_map[found_e] : found_e;
    const int row0 = A.bounds[be] + found_g * BN;
    const int nrows = min(BN, A.bounds[be + 1] - row0);
    const int m0 = (int) blockIdx.x * BM;
    const int K = A.w_cols, nkt = K / BK;
    const size_t rbw = row_bytes(T, K);
    const uint8_t* wexp = A.w + (size_t) found_e * A.expert_bytes;
    const size_t xrb = (size_t) (K / 32) * kQ81Bytes;

    constexpr int NA = GLU ? 2 : 1;
    constexpr int kStageBytes = (NA + 1) * kTileBytes;
    constexpr uint32_t kCols = GLU ? 256 : 128;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&s_done[s], 1);
        mbar_init(&s_final, 1);
        s_fail = 0;
    }
    mbar_fence_init();
    if (warp == 0) tmem_alloc(&s_tmem, kCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    constexpr uint32_t idesc = idesc_f16(BM, BN);

    const int r = tid & 127, h = tid >> 7;          // this thread's row of every tile and its 32-value half
    bool ok = true;
    for (int kt = 0; kt < nkt; ++kt) {
        const int s = kt % kStages;
        if (kt >= kStages && ok) {
            if (!mbar_wait(&s_done[s], ((kt / kStages) - 1) & 1)) ok = false;
        }
        uint8_t* stage = smem + (size_t) s * kStageBytes;
        float v[32];
        if (ok) {
#pragma unroll
            for (int a = 0; a < NA; ++a) {
                dequant32<T>(wexp + (size_t) (a * A.w_rows + m0 + r) * rbw, kt, h, v);
                store32(stage + a * kTileBytes, BM, r, 4 * h, v);
            }
            if (r < nrows) act32(A.xq + (size_t) (row0 + r) * xrb, kt, h, v);
            else {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = 0.0f;
            }
            store32(stage + NA * kTileBytes, BN, r, 4 * h, v);
        }
        fence_proxy_async();                         // my shared-memory writes before the tensor core's reads
        if (!ok) s_fail = 1;
        __syncthreads();
        if (s_fail) { ok = false; }
        if (tid == 0 && ok) {
            tc_fence_after();
            const uint32_t a_base = smem_u32(stage), b_base = smem_u32(stage + NA * kTileBytes);
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) {
                const uint64_t bd = smem_desc(b_base + kk * 2 * BN * 16, BN * 16, 128);
#pragma unroll
                for (int a = 0; a < NA; ++a) {
                    const uint64_t ad = smem_desc(a_base + a * kTileBytes + kk * 2 * BM * 16, BM * 16, 128);
                    mma_f16_ss(tmem + a * BN, ad, bd, idesc, (kt > 0 || kk > 0) ? 1u : 0u);
                }
            }
            mma_commit(&s_done[s]);
            if (kt == nkt - 1) mma_commit(&s_final);
        }
    }
    // ---- epilogue: warps 0..3 own the four 32-lane quadrants of tensor memory
    if (ok && !mbar_wait(&s_final, 0)) ok = false;
    tc_fence_after();
    if (ok && warp < 4) {
        const int m = m0 + 32 * warp + lane;         // this thread's weight row
        for (int c0 = 0; c0 < BN; c0 += 32) {
            if (c0 >= nrows) break;
            float g[32];
            tmem_ld32(tmem + ((uint32_t) (32 * warp) << 16) + c0, g);
            if constexpr (GLU) {
                float u[32];
                tmem_ld32(tmem + ((uint32_t) (32 * warp) << 16) + BN + c0, u);
#pragma unroll
                for (int j = 0; j < 32; ++j) g[j] = swiglu(g[j], u[j], A.limit);
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (c0 + j < nrows) {
                    const int row = row0 + c0 + j;
                    const int64_t drow = A.ids ? A.ids[row] : row;
                    A.dst[drow * A.ld_dst + m] = g[j];
                }
            }
        }
    }
    if (!ok && tid == 0 && A.error != nullptr) atomicExch(A.error, 1u);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kCols);
}

template<typename X>
__global__ void __launch_bounds__(256) mmq_quantize_kernel(const X* __restrict__ x, const int* __restrict__ ids,
                                                           uint8_t* __restrict__ xq, int64_t cols, int64_t ld,
                                                           int64_t n_blocks) {
    const int lane = threadIdx.x & 31;
    const int64_t b = (int64_t) blockIdx.x * 8 + (threadIdx.x >> 5);
    if (b >= n_blocks) return;
    const int64_t bpr = cols / 32, row = b / bpr, kb = b - row * bpr;
    const int64_t src = ids ? ids[row] : row;
    float v;
    if constexpr (sizeof(X) == 2) v = __uint_as_float((uint32_t) x[src * ld + kb * 32 + lane] << 16);   // bf16 bits, widened exactly
    else v = x[src * ld + kb * 32 + lane];
    q8_1_store_warp(v, xq + b * kQ81Bytes, lane);
}

template<typename X>
int launch_quantize(const X* x, const int32_t* ids, void* xq, int type, int64_t cols, int64_t ld, int64_t rows, void* stream) {
    if (!maya_mmq_supported(type)) return refuse(MAYA_ERR_TYPE);
    if (rows <= 0) return MAYA_OK;
    if (!x || !xq || cols <= 0 || cols % 32 || ld < cols) return refuse(MAYA_ERR_ARG);
    const int64_t nb = rows * (cols / 32);
    if ((nb + 7) / 8 > 0x7FFFFFFF) return refuse(MAYA_ERR_LIMIT);
    mmq_quantize_kernel<X><<<(unsigned) ((nb + 7) / 8), 256, 0, as_stream(stream)>>>(x, ids, (uint8_t*) xq, cols, ld, nb);
    return note_launch("mmq_quantize");
}

template<int T, bool GLU>
int launch_mmq(const MmqArgs& A, int64_t total_rows, cudaStream_t s) {
    constexpr size_t smem = (size_t) kStages * ((GLU ? 3 : 2) * kTileBytes);
    if (cudaFuncSetAttribute(mmq_kernel<T, GLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess)
        return note_launch("mmq smem attribute");
    const int64_t groups = total_rows / BN + A.n;     // an upper bound of sum(ceil(rows_e / 128)), known without the counts
    if (groups > 65535) return refuse(MAYA_ERR_LIMIT);
    const dim3 grid((unsigned) (A.w_rows / BM), (unsigned) groups);
    mmq_kernel<T, GLU><<<grid, kMmqThreads, smem, s>>>(A);
    return note_launch("mmq");
}

int run_product(const maya_mmq_product* p, bool glu, float limit, cudaStream_t s) {
    if (!p || !p->w || !p->xq || !p->bounds || !p->dst) return refuse(MAYA_ERR_ARG);
    if (p->type != MAYA_Q4_K && p->type != MAYA_Q8_0) return refuse(MAYA_ERR_TYPE);
    if (p->n <= 0 || p->total_rows <= 0) return MAYA_OK;
    const int64_t out_rows = glu ? p->w_rows / 2 : p->w_rows;
    if (p->w_cols <= 0 || p->w_cols % 256 || out_rows <= 0 || out_rows % BM || (glu && p->w_rows % 2)) return refuse(MAYA_ERR_ARG);
    if (p->expert_bytes % (size_t) type_bytes(p->type) || p->ld_dst < out_rows) {
        std::fprintf(stderr, "maya_mmq_run: expert_bytes %zu is not a whole number of blocks, or ld_dst too small\n", p->expert_bytes);
        return refuse(MAYA_ERR_ARG);
    }
    if (!aligned16(p->w) || p->expert_bytes % 16) return refuse(MAYA_ERR_ARG);
    MmqArgs A{};
    A.w = (const uint8_t*) p->w; A.expert_bytes = p->expert_bytes; A.w_rows = (int) out_rows; A.w_cols = (int) p->w_cols;
    A.n = p->n; A.expert_map = p->expert_map; A.xq = (const uint8_t*) p->xq; A.bounds = p->bounds; A.ids = p->ids;
    A.dst = p->dst; A.ld_dst = p->ld_dst; A.limit = limit; A.error = p->error;
    if (p->type == MAYA_Q4_K) return glu ? launch_mmq<MAYA_Q4_K, true>(A, p->total_rows, s) : launch_mmq<MAYA_Q4_K, false>(A, p->total_rows, s);
    return glu ? launch_mmq<MAYA_Q8_0, true>(A, p->total_rows, s) : launch_mmq<MAYA_Q8_0, false>(A, p->total_rows, s);
}

}  // namespace
}  // namespace maya

using namespace maya;

extern "C" int maya_mmq_supported(int type) { return type == MAYA_Q4_K || type == MAYA_Q8_0; }
extern "C" size_t maya_mmq_q8_bytes(int64_t rows, int64_t cols) {
    if (rows <= 0 || cols <= 0 || cols % 32) return 0;
    return (size_t) rows * (size_t) (cols / 32) * kQ81Bytes;
}
extern "C" int maya_mmq_quantize(const float* x, const int32_t* ids, void* xq, int type, int64_t cols, int64_t ld,
                                 int64_t rows, void* stream) {
    return launch_quantize<float>(x, ids, xq, type, cols, ld, rows, stream);
}
extern "C" int maya_mmq_quantize_bf16(const uint16_t* x, const int32_t* ids, void* xq, int type, int64_t cols, int64_t ld,
                                      int64_t rows, void* stream) {
    return launch_quantize<uint16_t>(x, ids, xq, type, cols, ld, rows, stream);
}
extern "C" int maya_mmq_run(const maya_mmq_product* p, void* stream) { return run_product(p, false, 0.0f, as_stream(stream)); }
extern "C" int maya_mmq_run_glu(const maya_mmq_product* p, float limit, void* stream) {
    return run_product(p, true, limit, as_stream(stream));
}
