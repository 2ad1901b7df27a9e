// moe_window.cu - the window path's down projection with its weight rows streamed through shared memory.
//
// down_groups_kernel (moe_decode.cu) reads a group's rows straight from global memory, one warp item at a time, and its
// warps wait on their own loads.  Here one 512-thread block an SM walks an even share of the window's work - items
// (group, pass of four of its columns, chunk of 64 rows) - and brings each item's rows (contiguous in the expert blob,
// 74 KB for Q4_K at n_ff = 2048) into a two-stage ring with cp.async.bulk one item ahead of the dot loops, which then
// read weights and activations from shared memory only: 107 against 116 us on the 8-token Q4_K window.  (The same
// form for gate/up - one weight row a warp, since a stage of 16 rows of n_embd values is all that fits twice - re-reads
// the activation blocks for every row and is slower than gate_up_kernel, 223 against 194 us; it is not built in.)
//
// The arithmetic is rows_dot<T, 4, NC>'s, value for value (the same decode, the same column loop, the same lane order),
// so every token's result stays bit-identical to the single-token kernels'.
//
// Plain bulk copies (one destination: this block) of this GPU's own memory; every wait is bounded, and a wait that runs out makes the
// block stop (its outputs are then missing) after the copies in flight were given the same bounded time to land.  A
// blob that is not 16-byte aligned (bulk copies need it) is copied with ordinary loads instead.
#include "maya_dots.cuh"
#include "maya_internal.cuh"
#include "maya_stream.cuh"

#include <atomic>

namespace maya {
namespace {

constexpr int kWNC = 4;            // activation columns per pass (as the group kernels)
constexpr int kWRows = 64;         // output rows per item: 16 warps x 4 rows
constexpr int kWWarps = 16;
constexpr int kWThreads = kWWarps * 32;
constexpr int kWMaxGroups = 128;   // T <= 16 tokens x 8 routes

struct WGroups {
    const unsigned long long* ptr;
    const int* start;
    const int* n_groups;
    const int* ent_slot;
    int cap;
    __device__ __forceinline__ int slot(int e) const { return ent_slot ? ent_slot[e] : e; }
};

struct WShared {
    uint64_t full[2];
    int cum[kWMaxGroups + 1];      // items before group g
    int fail;
};

// Item `it` of the window's list: its group, pass and chunk.  `g` is a cursor that only moves forward.
__device__ __forceinline__ void locate(const WShared& sh, int it, int nchunks, int& g, int& pass, int& chunk) {
    while (it >= sh.cum[g + 1]) ++g;
    const int r = it - sh.cum[g];
    pass = r / nchunks;
    chunk = r - pass * nchunks;
}

// part[slot][row] = down[row] . hq[slot] for every entry of every group (unweighted), rows of n_ff values
template<int T>
__global__ void __launch_bounds__(kWThreads, 1) down_stream_kernel(WGroups G, int n_embd, int n_ff, size_t down_off,
                                                                   const uint8_t* __restrict__ hq, float* __restrict__ part) {
    extern __shared__ __align__(128) uint8_t s_raw[];
    __shared__ WShared sh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t rb = row_bytes(T, n_ff);
    const int nchunks = (n_embd + kWRows - 1) / kWRows;
    const uint32_t stage_stride = ((uint32_t) (kWRows * rb) + 127u) & ~127u;
    auto st = [&](int s) -> uint8_t* { return s_raw + (size_t) s * stage_stride; };
    uint32_t* const s_tab = (uint32_t*) (s_raw + 2 * (size_t) stage_stride);
    int4* q; float* d; int* is;
    const int nblk = n_ff / 32;
    const XCols x = xcols_carve((uint8_t*) s_tab + Fmt<T>::tab_words * 4, nblk, kWNC, &q, &d, &is);
    const size_t hq_stride = (size_t) nblk * kQ81Bytes;

    // ---- the window's items and this block's share of them
    int ng = G.n_groups ? *G.n_groups : G.cap;
    ng = min(min(ng, G.cap), kWMaxGroups);
    if (tid == 0) {
        int run = 0;
        for (int g = 0; g < ng; ++g) {
            sh.cum[g] = run;
            const int ne = G.start[g + 1] - G.start[g];
            if (G.ptr[g] != 0ull && ne > 0) run += ((ne + kWNC - 1) / kWNC) * nchunks;
        }
        sh.cum[ng] = run;
        sh.fail = 0;
        mbar_init(&sh.full[0], 1);
        mbar_init(&sh.full[1], 1);
        mbar_fence_init();
    }
    load_tab<T>(s_tab);
    __syncthreads();
    const int total = sh.cum[ng];
    const int lo = (int) ((long long) blockIdx.x * total / gridDim.x), hi = (int) ((long long) (blockIdx.x + 1) * total / gridDim.x);
    if (hi <= lo) return;

    // the item's rows: where they are, how many, whether a bulk copy can bring them
    auto source = [&](int g, int chunk, const uint8_t*& src, int& nrows, bool& bulk) {
        nrows = min(kWRows, n_embd - chunk * kWRows);
        src = (const uint8_t*) G.ptr[g] + down_off + (size_t) chunk * kWRows * rb;
        bulk = ((((uintptr_t) src) | (uint32_t) (nrows * rb)) & 15u) == 0;
    };
    // thread 0: start the copy of item `it` into its stage (nothing to do for a blob that needs ordinary loads)
    int g_pf = 0;
    auto issue = [&](int it) {
        int pass, chunk, nrows;
        const uint8_t* src;
        bool bulk;
        locate(sh, it, nchunks, g_pf, pass, chunk);
        source(g_pf, chunk, src, nrows, bulk);
        if (!bulk) return;
        const int s = (it - lo) & 1;
        fence_proxy_async();                         // the stage's earlier readers (and writers, on the ordinary-load path) come first
        mbar_expect_tx(&sh.full[s], (uint32_t) (nrows * rb));
        bulk_load(st(s), src, (uint32_t) (nrows * rb), &sh.full[s]);
    };
    if (tid == 0) {
        issue(lo);
        if (lo + 1 < hi) issue(lo + 1);
    }

    int g = 0, cur_g = -1, cur_pass = -1;
    uint32_t ph = 0u;                                // bit s: the phase of full[s] to wait for next
    for (int it = lo; it < hi; ++it) {
        int pass, chunk, nrows;
        const uint8_t* src;
        bool bulk;
        locate(sh, it, nchunks, g, pass, chunk);
        source(g, chunk, src, nrows, bulk);
        const int s = (it - lo) & 1;
        const int e0 = G.start[g] + pass * kWNC, nc = min(kWNC, G.start[g + 1] - e0);
        if (g != cur_g || pass != cur_pass) {        // the pass's columns (the previous item's closing barrier freed the old ones)
            for (int c = 0; c < nc; ++c)
                xcols_stage_p<Dec<T>::xblk, T == MAYA_IQ1_S>(hq + (size_t) G.slot(e0 + c) * hq_stride, 0, nblk, 1, q + (size_t) 2 * c * nblk,
                                                             d + (size_t) c * nblk, is + (size_t) c * nblk);
            cur_g = g;
            cur_pass = pass;
            __syncthreads();
        }
        bool ok = true;
        if (bulk) {
            ok = mbar_wait(&sh.full[s], (ph >> s) & 1u);      // bounded
            if (ok) ph ^= 1u << s;
            else sh.fail = 1;
        } else {                                     // ordinary loads, everyone
            const uint32_t bytes = (uint32_t) (nrows * rb);
            for (uint32_t i = tid * 2; i < bytes; i += kWThreads * 2) *(uint16_t*) (st(s) + i) = *(const uint16_t*) (src + i);
            __syncthreads();
        }
        const int rl = warp * 4;                     // this warp's four rows of the item
        if (ok && rl < nrows) {
            const uint8_t* rows[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) rows[j] = st(s) + (size_t) min(rl + j, nrows - 1) * rb;
            float o[4][kWNC];
            rows_dot<T, 4, kWNC>(rows, x, nc, n_ff, lane, s_tab, o);
            if (lane == 0) {
#pragma unroll
                for (int c = 0; c < kWNC; ++c) {
                    if (c >= nc) continue;
                    float* out = part + (size_t) G.slot(e0 + c) * n_embd + chunk * kWRows + rl;
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (rl + j < nrows) out[j] = o[j][c];
                }
            }
        }
        __syncthreads();                             // everyone is done with stage s (and with the columns, if they change next)
        if (sh.fail) break;                          // the same for every thread
        if (tid == 0 && it + 2 < hi) issue(it + 2);
    }
    if (sh.fail) {
        // let what may still be in flight land (bounded as well) before the block's shared memory goes away
        mbar_wait(&sh.full[0], ph & 1u);
        mbar_wait(&sh.full[1], (ph >> 1) & 1u);
    }
}

template<int T> size_t stream_smem(int n_ff) {
    const size_t stage = ((size_t) kWRows * row_bytes(T, n_ff) + 127) & ~(size_t) 127;
    return 2 * stage + (size_t) Fmt<T>::tab_words * 4 + xcols_bytes(n_ff / 32, kWNC);
}

int sm_count() {
    static std::atomic<int> cached_dev{-1}, cached_n{0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (cached_dev.load() != dev) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        cached_n.store(n);
        cached_dev.store(dev);
    }
    return cached_n.load();
}

template<int T>
int launch_stream(const WGroups& G, int n_embd, int n_ff, size_t down_off, const void* hq, float* part, cudaStream_t s) {
    const size_t smem = stream_smem<T>(n_ff);
    static std::atomic<size_t> set_for{0};            // per instantiation: the size the attribute was last raised to
    static std::atomic<int> set_dev{-1};
    int dev = 0;
    cudaGetDevice(&dev);
    if (set_dev.load() != dev || set_for.load() < smem) {
        if (cudaFuncSetAttribute(down_stream_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess)
            return note_launch("down_window_stream smem attribute");
        set_dev.store(dev);
        set_for.store(smem);
    }
    const int blocks = sm_count();
    if (blocks <= 0) return refuse(MAYA_ERR_ARG);
    down_stream_kernel<T><<<blocks, kWThreads, smem, s>>>(G, n_embd, n_ff, down_off, (const uint8_t*) hq, part);
    return note_launch("down_window_stream");
}

constexpr size_t kStreamSmemMax = 200 * 1024;

}  // namespace

// Whether down_stream_kernel covers the shapes: an item's 64 rows must fit shared memory twice beside the staged columns
// and be a whole number of 16-byte words.
bool window_down_stream_supported(int d_type, int T, int n_ff) {
    if (T * 8 > kWMaxGroups) return false;
    size_t b = 0;
    switch (d_type) {
        case MAYA_Q8_0: b = stream_smem<MAYA_Q8_0>(n_ff); break;
        case MAYA_Q4_K: b = stream_smem<MAYA_Q4_K>(n_ff); break;
        case MAYA_IQ2_S: b = stream_smem<MAYA_IQ2_S>(n_ff); break;
        case MAYA_IQ3_S: b = stream_smem<MAYA_IQ3_S>(n_ff); break;
        default: return false;
    }
    return (kWRows * row_bytes(d_type, n_ff)) % 16 == 0 && b <= kStreamSmemMax;
}

// The down projection of a window's groups (the arrays maya_moe_win_group fills): hq [slot] -> part [slot][n_embd].
int window_down_stream(int d_type, const maya_moe_win* w, cudaStream_t s) {
    WGroups G{w->grp_ptr, w->grp_start, w->n_groups, w->grp_ent, w->T * 8};
#define MAYA_WDN(TT) case TT: return launch_stream<TT>(G, w->n_embd, w->n_ff, w->down_off, w->hq, w->part, s);
    switch (d_type) {
        MAYA_WDN(MAYA_Q8_0) MAYA_WDN(MAYA_Q4_K) MAYA_WDN(MAYA_IQ2_S) MAYA_WDN(MAYA_IQ3_S)
        default: return refuse(MAYA_ERR_TYPE);
    }
#undef MAYA_WDN
}

}  // namespace maya
