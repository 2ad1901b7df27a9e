// mmq_tc.cu - the prompt path's grouped-by-expert GEMM over quantized expert matrices on the 5th-generation tensor
// cores: for every expert e, the activation rows [bounds[e], bounds[e+1]) times its [w_rows, w_cols] quantized matrix.
//
// Replaces mmq::quantize / mmq::Context::run / run_glu (include/strata/prefill/moe_mmq.hpp:34-81, src/prefill/
// moe_mmq.cu:114-228), which wrap llama.cpp's int8 `mma.sync` MMQ kernels (not part of the reference tree).  The
// reference rounds activations to q8_1 and multiplies integers with per-32 scales; an integer tcgen05 contraction
// would have to leave tensor memory every 32 values of K to apply those scales, so here both operands are f16:
// activations are stored once as d * q of their q8_1 image (the reference's rounding of x, kept so that results stay
// within its tolerance), weights are expanded from their GGUF blocks in shared memory, and `tcgen05.mma.kind::f16`
// accumulates in f32 in tensor memory.
//
// One block = a slab of 256 weight rows (128 gate + 128 up rows for the fused SwiGLU form) x up to 160 activation
// rows of one expert: two M = 128 accumulators of N = rows (rounded up to 16) columns in tensor memory.  The expanded
// weights are the A operand and live in tensor memory too (lane = weight row, the layout a thread-per-row expansion
// produces by itself), so shared memory carries only raw blocks and activations: an SM's 128 bytes/clock of shared
// memory cannot feed two f16 operands of M = N = 128 products at the tensor core's rate.  Warp roles:
//   warp 16     one lane: TMA loads of raw weight blocks, 64 rows x 256 K-values a "unit", into a ring of units;
//   warp 18     one lane: TMA loads of activation tiles, 128 (+ 32) rows x 64 K-values, in the 128-byte swizzle layout
//               the tensor core reads at full rate;
//   warps 0..15 two teams of 8 warps that take alternate K steps; in a team one thread per weight row expands 32
//               K-values of the row per step (packed half2 arithmetic: Q8_0 w = q * d; Q4_K w = fma(q, d * sc,
//               -(dmin * m))) and tcgen05.st-s them into the row's lane;
//   warps 17,19 one lane each, one accumulator each: two tcgen05.mma per step (2 K = 16 halves, A from tensor memory,
//               B from shared memory), one commit per two steps -> the steps' buffers are free (a single thread
//               cannot issue products as fast as the tensor core retires them unless its loop is a few instructions);
//   warps 0..15 afterwards: the epilogue - tcgen05.ld (lane = weight row, column = activation row), SwiGLU, optional
//               q8_1 rounding of h for the next product, then through shared memory: one bulk copy per activation row.
// Which expert and which 160-row group of it a block handles is found on the device from `bounds`; no count travels
// to the host.  Every mbarrier wait is bounded: a wait that runs out sets the error word, the roles stop, copies in
// flight are waited for (bounded), tensor memory is freed and the block returns.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_fp16.h>

#include <cstdio>
#include <cstring>

#include "maya_internal.cuh"
#include "maya_tcgen05.cuh"

namespace maya {
namespace {

constexpr int TM = 256;                 // weight rows of a block
constexpr int TN = 160;                 // most activation rows of a block
constexpr int BK = 32;                  // K values of one step
constexpr int kSt = 3;                  // stages of expanded weights (the A operand, in tensor memory), 64 K-values each
constexpr int kUnitRows = 64;           // weight rows of one raw unit
constexpr int kDqWarps = 16;            // two teams of 8
constexpr int kMmqThreads = (kDqWarps + 4) * 32;   // + raw-unit loader, issuer of accumulator 0, activation loader, issuer of accumulator 1
constexpr int kBBox = 128 * 64 * 2;     // 16 KB: 128 activation rows x 64 K-values, 128-byte swizzle
constexpr int kBStage = kBBox + 32 * 64 * 2;   // + the 32-row box of a block with more than 128 rows: 20 KB
constexpr uint32_t kAccCols = TN;       // tensor-memory columns: accumulator 0 at 0, accumulator 1 at 160,
constexpr uint32_t kACol = 2 * TN;      // the A operand's 3 stages from 320: per stage 32 columns for each accumulator
constexpr int kMaxUnits = 16;
constexpr int kDone = 16;               // ring of "pair of K steps consumed" barriers (one tcgen05.commit per pair: a commit
                                        // costs the tensor pipe about as much as a product)
// Raw weight units, one tiled TMA box of 64 rows each.  Q8_0 / Q4_K: a row's 256 K-values are 272 / 144 bytes, a
// multiple of 16.  IQ2_S / IQ3_S blocks are 82 / 110 bytes: the box is the 16-byte aligned window around the rows' block
// (96 / 128 bytes used) taken 112 / 144 bytes wide, so that rows are an odd number of 16-byte words apart in shared
// memory (a warp's 16-byte reads of 32 rows fall in different banks).
template<int T> constexpr bool kIq = T == MAYA_IQ2_S || T == MAYA_IQ3_S;
template<int T> constexpr int kBlkBytes = T == MAYA_IQ2_S ? 82 : T == MAYA_IQ3_S ? 110 : 0;
template<int T> constexpr int kWin = T == MAYA_IQ2_S ? 96 : 128;
template<int T> constexpr int kRawRow = T == MAYA_Q4_K ? 144 : T == MAYA_Q8_0 ? 272 : T == MAYA_IQ2_S ? 112 : 144;
template<int T> constexpr int kUnitBytes = kUnitRows * kRawRow<T>;
template<int T> constexpr int kUnits = T == MAYA_Q4_K ? 10 : T == MAYA_Q8_0 ? 8 : T == MAYA_IQ2_S ? 14 : 12;   // raw units in flight
template<int T> constexpr int kBStages = T == MAYA_Q4_K ? 6 : 4;            // activation tiles (64 K-values) in flight
template<int T> constexpr int kBRing = kBStages<T> * kBStage;
// i-quants: the codebook as f16 (IQ2_S 1024 x 8 values, IQ3_S 512 x 4 values) and the 256 sign patterns as f16 sign masks
template<int T> constexpr int kGridBytes = T == MAYA_IQ2_S ? 1024 * 16 : T == MAYA_IQ3_S ? 512 * 8 : 0;
template<int T> constexpr int kTabBytes = kIq<T> ? kGridBytes<T> + 256 * 16 : 0;
template<int T> constexpr int kTabOff = kBRing<T> + kUnits<T> * kUnitBytes<T>;
template<int T> constexpr size_t kSmemBytes = (size_t) kTabOff<T> + kTabBytes<T>;
static_assert(kUnits<MAYA_Q4_K> <= kMaxUnits && kUnits<MAYA_Q8_0> <= kMaxUnits && kUnits<MAYA_IQ2_S> <= kMaxUnits &&
              kUnits<MAYA_IQ3_S> <= kMaxUnits, "one mbarrier pair per raw unit");

// The activation image: a row is its w_cols f16 values d * q, then one f16 per 32 values - the group's SUM CORRECTION
// xa = f16(sum of the unquantized values) - sum of the row's stored d * q values - padded with zeros to a multiple of 64.  llama.cpp's
// MMQ keeps that unquantized sum beside the block (the "ds4" q8_1 layout) and a type with a constant term per group
// (Q4_K: -dmin * m) multiplies the term by it, not by the sum of the rounded values; here the same result comes from
// extra K steps inside a Q4_K product: A = -dmin * m of a row's groups, B = xa.  Other types do not read the tail.
// Optional clock stamps of a tile's phases (built only with -DMAYA_MMQ_STAMPS, see build.py --stamps and
// mmq_tile_phases.py): 16 slots per tile for the first 4096 tiles of each of the four (type class, fused) kernels.
#ifdef MAYA_MMQ_STAMPS
__device__ long long g_stamps[4 * 4096 * 16];
#define MAYA_STAMP(i) do { if (stamp_id >= 0) stamps[(i)] = clock64(); } while (0)
#else
#define MAYA_STAMP(i) do { } while (0)
#endif
__host__ __device__ constexpr int64_t xq_tail(int64_t cols) { return ((cols / 32) + 63) & ~(int64_t) 63; }
__host__ __device__ constexpr int64_t xq_ld(int64_t cols) { return cols + xq_tail(cols); }

struct MmqArgs {
    const uint8_t* w;            // the matrices (the i-quant path copies row windows itself; the others go through tm_w)
    size_t expert_bytes;
    int mat_rows;                // rows of one matrix (2 n_ff for the fused form)
    int w_rows, w_cols;          // rows of one output (n_ff for the fused form: gate rows, then up rows), K
    int n;                       // matrices of this product
    const int* expert_map;       // optional: matrix i owns the rows of bounds entry expert_map[i]
    const int* bounds;
    const int* ids;              // optional dst row of a sorted row
    float* dst;                  // optional for the fused form
    int64_t ld_dst;
    __half* xq_out;              // fused form, optional: q8_1-rounded h as f16, [sorted row][w_rows]
    float limit;
    unsigned* error;             // optional sticky error word
};

__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *(uint32_t*) &h; }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *(__half2*) &u; }
// bytes (lo, hi) of x -> the half2 (1024 + lo, 1024 + hi): 0x64 is the high byte of 1024.0 in f16
__device__ __forceinline__ __half2 bytes01_plus1024(uint32_t x) { return bits_h2(__byte_perm(x, 0x64646464u, 0x4140)); }
__device__ __forceinline__ __half2 bytes23_plus1024(uint32_t x) { return bits_h2(__byte_perm(x, 0x64646464u, 0x4342)); }

// The q8_1 rounding of maya_mmq_quantize for a thread that holds 8 consecutive values of a 32-value group (the group's
// four threads are four consecutive lanes; every lane of the warp must call): llama.cpp's quantize_mmq_q8_1 as the
// reference's host model states it - d_inv = 127 / amax, q = round(v * d_inv) clamped to +-127, d = min(1 / d_inv, 65504)
// kept as f16, stored f16(d) * q.  o = the 8 stored values; the return value is the group's sum correction
// f16(S) - sum of the stored values, with S added in quantize_mmq_q8_1's order: four consecutive values left to right
// (this thread holds partial sums 2j and 2j + 1 of the group's eight), then the tree at distances 4, 2, 1.
__device__ __forceinline__ __half q8_1_round8(const float (&v)[8], uint32_t (&o)[4]) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    const float d_inv = __fdiv_rn(127.0f, amax);
    const float dh = amax == 0.0f ? 0.0f : __half2float(__float2half_rn(fminf(__fdiv_rn(1.0f, d_inv), 65504.0f)));
    float bsum = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float q0 = 0.0f, q1 = 0.0f;
        if (amax != 0.0f) {
            q0 = fmaxf(-127.0f, fminf(127.0f, roundf(__fmul_rn(v[2 * i], d_inv))));
            q1 = fmaxf(-127.0f, fminf(127.0f, roundf(__fmul_rn(v[2 * i + 1], d_inv))));
        }
        const __half2 r = __floats2half2_rn(dh * q0, dh * q1);
        o[i] = h2_bits(r);
        bsum += __low2float(r) + __high2float(r);     // the stored values: multiples of one power of two, 24 bits in all - exact
    }
    float s0 = __fadd_rn(__fadd_rn(__fadd_rn(v[0], v[1]), v[2]), v[3]), s1 = __fadd_rn(__fadd_rn(__fadd_rn(v[4], v[5]), v[6]), v[7]);
    s0 = __fadd_rn(s0, __shfl_xor_sync(0xFFFFFFFFu, s0, 2));
    s1 = __fadd_rn(s1, __shfl_xor_sync(0xFFFFFFFFu, s1, 2));
    s0 = __fadd_rn(s0, __shfl_xor_sync(0xFFFFFFFFu, s0, 1));
    s1 = __fadd_rn(s1, __shfl_xor_sync(0xFFFFFFFFu, s1, 1));
    bsum += __shfl_xor_sync(0xFFFFFFFFu, bsum, 1);
    bsum += __shfl_xor_sync(0xFFFFFFFFu, bsum, 2);
    return __float2half_rn(__half2float(__float2half_rn(__fadd_rn(s0, s1))) - bsum);
}

// ---- Q4_K: the 16-byte header of a 144-byte block -> d * sc and -(dmin * m) of its 8 sub-blocks, as half2 pairs
struct Q4Scales { __half2 dl[8], nml[8]; };
__device__ __forceinline__ void q4k_scales(const uint4 hdr, Q4Scales& S) {
    const __half2 dd = bits_h2(hdr.x);
    const __half2 d2 = __low2half2(dd), m2 = __high2half2(dd);
    const uint32_t s[3] = {hdr.y, hdr.z, hdr.w};
    auto byte = [&](int i) -> uint32_t { return (s[i >> 2] >> (8 * (i & 3))) & 0xFF; };
    const __half2 k1024 = __float2half2_rn(1024.0f);
#pragma unroll
    for (int sb = 0; sb < 8; ++sb) {
        uint32_t sc, mn;
        if (sb < 4) { sc = byte(sb) & 63; mn = byte(sb + 4) & 63; }
        else { sc = (byte(sb + 4) & 0x0F) | ((byte(sb - 4) >> 6) << 4); mn = (byte(sb + 4) >> 4) | ((byte(sb) >> 6) << 4); }
        const __half2 sc2 = __hsub2(bits_h2(0x64006400u | sc | (sc << 16)), k1024);      // exact
        const __half2 mn2 = __hsub2(bits_h2(0x64006400u | mn | (mn << 16)), k1024);
        S.dl[sb] = __hmul2(d2, sc2);
        S.nml[sb] = __hneg2(__hmul2(m2, mn2));
    }
}
// 32 weights of sub-block (2p + hi) from the 32 quant bytes of pair p
__device__ __forceinline__ void q4k_stage(const uint4 qa, const uint4 qb, int hi, __half2 dl, __half2 nml, uint32_t* r) {
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    const __half2 k1024 = __float2half2_rn(1024.0f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t x = (hi ? (w[i] >> 4) : w[i]) & 0x0F0F0F0Fu;
        r[2 * i] = h2_bits(__hfma2(__hsub2(bytes01_plus1024(x), k1024), dl, nml));
        r[2 * i + 1] = h2_bits(__hfma2(__hsub2(bytes23_plus1024(x), k1024), dl, nml));
    }
}
// ---- Q8_0: block J (34 bytes) of a 272-byte raw row, read as three aligned 16-byte words
template<int J>
__device__ __forceinline__ void q80_stage(const uint8_t* rrow, uint32_t* r) {
    constexpr int kBase = (34 * J) / 16 * 16, kOff = 34 * J - kBase;     // kOff = 0, 2, ..., 14
    const uint4 a = *(const uint4*) (rrow + kBase), b = *(const uint4*) (rrow + kBase + 16), c = *(const uint4*) (rrow + kBase + 32);
    const uint32_t w[12] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w, c.x, c.y, c.z, c.w};
    const uint32_t dw = w[kOff / 4];
    const __half dh = __ushort_as_half((unsigned short) ((kOff % 4) ? (dw >> 16) : (dw & 0xFFFF)));
    const __half2 d2 = __half2half2(dh), k1152 = __float2half2_rn(1152.0f);
    constexpr int kQ = kOff + 2;
    if constexpr (kQ % 4 != 0) {
        // the quants start two bytes into a word: values (4i, 4i + 1) are bytes 2, 3 of word i and values (4i + 2, 4i + 3)
        // bytes 0, 1 of word i + 1 - picked by the same byte permutes that widen them, no aligning permute
        uint32_t u[9];
#pragma unroll
        for (int i = 0; i < 9; ++i) u[i] = w[kQ / 4 + i] ^ 0x80808080u;     // q + 128 as unsigned bytes
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            r[2 * i] = h2_bits(__hmul2(__hsub2(bytes23_plus1024(u[i]), k1152), d2));
            r[2 * i + 1] = h2_bits(__hmul2(__hsub2(bytes01_plus1024(u[i + 1]), k1152), d2));
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t x = w[kQ / 4 + i] ^ 0x80808080u;
            r[2 * i] = h2_bits(__hmul2(__hsub2(bytes01_plus1024(x), k1152), d2));
            r[2 * i + 1] = h2_bits(__hmul2(__hsub2(bytes23_plus1024(x), k1152), d2));
        }
    }
}

// ---- i-quants.  `w` = the row's window as 32-bit words; the block starts OFF bytes into it (OFF is even and the same
// for all rows of a K block: every field position is a compile-time constant).
template<int BYTE> __device__ __forceinline__ uint32_t win_u32(const uint32_t* w) {
    constexpr int i = BYTE / 4, r = BYTE % 4;
    if constexpr (r == 0) return w[i];
    else if constexpr (r == 1) return __byte_perm(w[i], w[i + 1], 0x4321);
    else if constexpr (r == 2) return __byte_perm(w[i], w[i + 1], 0x5432);
    else return __byte_perm(w[i], w[i + 1], 0x6543);
}
template<int BYTE> __device__ __forceinline__ uint32_t win_u8(const uint32_t* w) { return (w[BYTE / 4] >> (8 * (BYTE % 4))) & 0xFF; }
template<int BYTE> __device__ __forceinline__ float win_f16(const uint32_t* w) {
    return __half2float(__ushort_as_half((unsigned short) ((w[BYTE / 4] >> (8 * (BYTE % 4))) & 0xFFFF)));
}
// IQ2_S (ggml dequantize_row_iq2_s): sub-block ib32 of 32 values: y = d (0.5 + ls) 0.25 * grid[qs | qh bits] * sign;
// here dl = f16(d (2 ls + 1) / 8) and w = dl * grid (one more f16 rounding), the sign XOR-ed into dl.
template<int OFF, int PP>
__device__ __forceinline__ void iq2s_pair(const uint32_t* w, const uint4* grid, const uint4* sgn, uint32_t* o) {
    const float d = win_f16<OFF>(w);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int ib = 2 * PP + h;
        const uint32_t qs4 = h ? win_u32<OFF + 2 + 4 * (2 * PP + 1)>(w) : win_u32<OFF + 2 + 4 * (2 * PP)>(w);
        const uint32_t sg4 = h ? win_u32<OFF + 34 + 4 * (2 * PP + 1)>(w) : win_u32<OFF + 34 + 4 * (2 * PP)>(w);
        const uint32_t qh = h ? win_u8<OFF + 66 + 2 * PP + 1>(w) : win_u8<OFF + 66 + 2 * PP>(w);
        const uint32_t sc = h ? win_u8<OFF + 74 + 2 * PP + 1>(w) : win_u8<OFF + 74 + 2 * PP>(w);
        (void) ib;
        const uint32_t dl0 = h2_bits(__float2half2_rn(d * (float) (2 * (sc & 15) + 1) * 0.125f));
        const uint32_t dl1 = h2_bits(__float2half2_rn(d * (float) (2 * (sc >> 4) + 1) * 0.125f));
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const uint32_t idx = ((qs4 >> (8 * l)) & 0xFF) | ((qh << (8 - 2 * l)) & 0x300);
            const uint4 G = grid[idx], M = sgn[(sg4 >> (8 * l)) & 0xFF];
            const uint32_t dl = l < 2 ? dl0 : dl1;
            uint32_t* r = o + 16 * h + 4 * l;
            r[0] = h2_bits(__hmul2(bits_h2(G.x), bits_h2(dl ^ M.x)));
            r[1] = h2_bits(__hmul2(bits_h2(G.y), bits_h2(dl ^ M.y)));
            r[2] = h2_bits(__hmul2(bits_h2(G.z), bits_h2(dl ^ M.z)));
            r[3] = h2_bits(__hmul2(bits_h2(G.w), bits_h2(dl ^ M.w)));
        }
    }
}
// IQ3_S (ggml dequantize_row_iq3_s): y = d (1 + 2 scale) * grid[qs | qh bit] * sign; 4 values per codebook entry.
template<int OFF, int PP>
__device__ __forceinline__ void iq3s_pair(const uint32_t* w, const uint2* grid, const uint4* sgn, uint32_t* o) {
    const float d = win_f16<OFF>(w);
    const uint32_t scb = win_u8<OFF + 106 + PP>(w);                    // scales[ib32 / 2]: low nibble ib32 even, high odd
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t q0 = h ? win_u32<OFF + 2 + 8 * (2 * PP + 1)>(w) : win_u32<OFF + 2 + 8 * (2 * PP)>(w);
        const uint32_t q1 = h ? win_u32<OFF + 6 + 8 * (2 * PP + 1)>(w) : win_u32<OFF + 6 + 8 * (2 * PP)>(w);
        const uint32_t qh = h ? win_u8<OFF + 66 + 2 * PP + 1>(w) : win_u8<OFF + 66 + 2 * PP>(w);
        const uint32_t sg4 = h ? win_u32<OFF + 74 + 4 * (2 * PP + 1)>(w) : win_u32<OFF + 74 + 4 * (2 * PP)>(w);
        const uint32_t nib = h ? (scb >> 4) : (scb & 15);
        const uint32_t db = h2_bits(__float2half2_rn(d * (float) (1 + 2 * nib)));
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const uint32_t q = l < 2 ? q0 : q1;
            const uint32_t i1 = ((q >> (16 * (l & 1))) & 0xFF) | ((qh << (8 - 2 * l)) & 256);
            const uint32_t i2 = ((q >> (16 * (l & 1) + 8)) & 0xFF) | ((qh << (7 - 2 * l)) & 256);
            const uint2 G1 = grid[i1], G2 = grid[i2];
            const uint4 M = sgn[(sg4 >> (8 * l)) & 0xFF];
            uint32_t* r = o + 16 * h + 4 * l;
            r[0] = h2_bits(__hmul2(bits_h2(G1.x), bits_h2(db ^ M.x)));
            r[1] = h2_bits(__hmul2(bits_h2(G1.y), bits_h2(db ^ M.y)));
            r[2] = h2_bits(__hmul2(bits_h2(G2.x), bits_h2(db ^ M.z)));
            r[3] = h2_bits(__hmul2(bits_h2(G2.y), bits_h2(db ^ M.w)));
        }
    }
}

struct Pipe {                       // static shared memory of a block
    uint64_t a_full[kSt], b_full[6];
    uint64_t done[kDone];            // done[p % kDone]: the products of K-step pair p (64 K-values) have completed
    uint64_t raw_full[kMaxUnits], raw_empty[kMaxUnits];
    uint64_t final;
    uint32_t tmem;
    int fail;
    int scan[2];                     // the block's (matrix, row group), found by warp 0
};

__device__ __forceinline__ bool failed(const Pipe& P) { return *(volatile const int*) &P.fail != 0; }
// Bounded wait; false when this wait ran out (the block's failure flag is then set) or another role has failed.
// (try_wait with a suspend-time hint, so that the waiting single-lane roles poll less, changed nothing when only the
// loaders used it and cost 0.7 % when the issuers and the expanding warps did.)
__device__ __forceinline__ bool wait_or_fail(Pipe& P, uint64_t* bar, uint32_t parity) {
    for (unsigned i = 0; i < (1u << 21); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 4096) {                          // try_wait itself suspends the thread for a while; back off only late
            __nanosleep(64);
            if ((i & 255) == 0 && failed(P)) return false;
        }
    }
    *(volatile int*) &P.fail = 1;
    return false;
}

template<int T, bool GLU>
__global__ void __launch_bounds__(kMmqThreads, 1)
mmq_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
           const __grid_constant__ CUtensorMap tm_x32, const MmqArgs A) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ Pipe P;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int NU = kUnits<T>, NB = kBStages<T>;

    // ---- which (matrix, 160-row group) is blockIdx.y: ONE warp scans the per-matrix group counts (each lane the counts
    //      of a run of consecutive matrices, an exclusive warp scan of the runs' sums, then the lane whose run holds the
    //      wanted group walks it), 1024 matrices a round, and leaves the answer in shared memory - one block barrier
    //      instead of the twenty a block-wide scan needs, on a path every tile and every surplus block of the grid takes
    if (warp == 0) {
        int found_e = -1, found_g = 0, base = 0;
        const int want_all = (int) blockIdx.y;
        for (int e0 = 0; e0 < A.n && found_e < 0; e0 += 1024) {
            const int per = (min(A.n - e0, 1024) + 31) >> 5;          // matrices a lane (<= 32)
            const int lo = e0 + lane * per, hi = min(lo + per, min(A.n, e0 + 1024));
            int mine = 0;
            for (int e = lo; e < hi; ++e) {
                const int be = A.expert_map ? A.expert_map[e] : e;
                mine += (A.bounds[be + 1] - A.bounds[be] + TN - 1) / TN;
            }
            int incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if (lane >= o) incl += v;
            }
            const int total = __shfl_sync(0xFFFFFFFFu, incl, 31);
            const int want = want_all - base;
            const unsigned holds = __ballot_sync(0xFFFFFFFFu, want >= incl - mine && want < incl);
            if (want < total && holds != 0u && lane == __ffs(holds) - 1) {
                int g = want - (incl - mine);
                for (int e = lo; e < hi; ++e) {
                    const int be = A.expert_map ? A.expert_map[e] : e;
                    const int cnt = (A.bounds[be + 1] - A.bounds[be] + TN - 1) / TN;
                    if (g < cnt) { found_e = e; found_g = g; break; }
                    g -= cnt;
                }
                P.scan[0] = found_e;
                P.scan[1] = found_g;
            }
            found_e = __shfl_sync(0xFFFFFFFFu, found_e, holds != 0u && want < total ? __ffs(holds) - 1 : 0);
            base += total;
        }
        if (found_e < 0 && lane == 0) P.scan[0] = -1;
    }
    __syncthreads();
    const int found_e = P.scan[0], found_g = P.scan[1];
    if (found_e < 0) return;                        // beyond the last group: uniform for the whole block
    const int be = A.expert_map ? A.expert_map[found_e] : found_e;
    const int row0 = A.bounds[be] + found_g * TN;
    const int nrows = min(TN, A.bounds[be + 1] - row0);
    const bool big = nrows > 128;                   // the activation tile is a 128-row box and a 32-row box
    const int m0 = (int) blockIdx.x * (GLU ? 128 : TM);
    const int nkt = A.w_cols / BK, nkb = A.w_cols / 256;
    // Q4_K: after every 8 blocks of K (32 pairs of K steps) one more pair carries the sum correction of those blocks' 64
    // groups - A = the groups' constant terms -dmin * m, B = the tail of the activation image (see xq_tail); the last pair
    // of a K that is not a multiple of 2048 is padded with zeros.  ntp = how many such pairs.
    const int ntp = T == MAYA_Q4_K ? (nkb + 7) / 8 : 0;
#ifdef MAYA_MMQ_STAMPS
    const int stamp_lin = (int) (blockIdx.y * gridDim.x + blockIdx.x);
    const int stamp_id = stamp_lin < 4096 ? stamp_lin : -1;
    long long* const stamps = g_stamps + ((size_t) ((T == MAYA_Q4_K || T == MAYA_IQ3_S ? 2 : 0) + (GLU ? 1 : 0)) * 4096 + max(stamp_id, 0)) * 16;
    if (tid == 0 && stamp_id >= 0) { stamps[0] = clock64(); stamps[14] = nrows; stamps[15] = nkt / 2 + ntp; }
#endif

    uint8_t* const raw = smem + kBRing<T>;
    if (tid == 0) {
        for (int s = 0; s < kSt; ++s) mbar_init(&P.a_full[s], 8);
        for (int s = 0; s < NB; ++s) mbar_init(&P.b_full[s], 1);
        for (int s = 0; s < kDone; ++s) mbar_init(&P.done[s], 2);      // both issuers commit
        for (int u = 0; u < NU; ++u) { mbar_init(&P.raw_full[u], 1); mbar_init(&P.raw_empty[u], 4); }
        mbar_init(&P.final, 2);
        P.fail = 0;
    }
    if constexpr (kIq<T>) {                         // the codebook as f16 and the sign masks, once per block
        uint4* sgn = (uint4*) (smem + kTabOff<T> + kGridBytes<T>);
        for (int i = tid; i < 256; i += kMmqThreads) {
            uint4 m;
            const uint32_t b = (uint32_t) i;       // bit j of the pattern: value j is negative; two values per f16 pair
            m.x = ((b & 1u) << 15) | ((b & 2u) << 30);
            m.y = ((b & 4u) << 13) | ((b & 8u) << 28);
            m.z = ((b & 16u) << 11) | ((b & 32u) << 26);
            m.w = ((b & 64u) << 9) | ((b & 128u) << 24);
            sgn[i] = m;
        }
        const __half2 k1024 = __float2half2_rn(1024.0f);
        if constexpr (T == MAYA_IQ2_S) {
            uint4* grid = (uint4*) (smem + kTabOff<T>);
            for (int i = tid; i < 1024; i += kMmqThreads) {
                const uint2 g = ((const uint2*) g_iq2s_grid)[i];
                uint4 v;
                v.x = h2_bits(__hsub2(bytes01_plus1024(g.x), k1024)); v.y = h2_bits(__hsub2(bytes23_plus1024(g.x), k1024));
                v.z = h2_bits(__hsub2(bytes01_plus1024(g.y), k1024)); v.w = h2_bits(__hsub2(bytes23_plus1024(g.y), k1024));
                grid[i] = v;
            }
        } else {
            uint2* grid = (uint2*) (smem + kTabOff<T>);
            for (int i = tid; i < 512; i += kMmqThreads) {
                const uint32_t g = g_iq3s_grid[i];
                uint2 v;
                v.x = h2_bits(__hsub2(bytes01_plus1024(g), k1024)); v.y = h2_bits(__hsub2(bytes23_plus1024(g), k1024));
                grid[i] = v;
            }
        }
    }
    mbar_fence_init();
    if (warp == 0) tmem_alloc(&P.tmem, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = P.tmem;
    if (tid == 0) MAYA_STAMP(1);                    // set-up done

    if (warp < kDqWarps) {
        // ------------------------------------------------------------ weight expansion
        // Two teams of 8 warps; in each, thread = one of the slab's 256 rows.  Team t expands the K steps kt with
        // kt % 2 == t, so that a step's latency (shared-memory reads, the packed-half chain, the tensor-memory store
        // and its wait) overlaps the other team's step.
        const int team = warp >> 3, row = tid & 255, w8 = warp & 7;
        const int slab = row >> 6;
        const uint8_t* const rbase = raw + (size_t) (row & 63) * kRawRow<T>;
        // rows 0..127 feed accumulator 0, rows 128..255 accumulator 1; a warp reaches the 32 lanes of its quadrant
        const uint32_t a_lane = tmem + ((uint32_t) (32 * (w8 & 3)) << 16) + kACol + (w8 >> 2) * 32;
        bool ok = true;
        auto put = [&](int kp, const uint32_t (&o)[32]) -> bool {   // the row's 64 values of pair kp -> its lane
            const int s = kp % kSt;
            if (kp >= kSt) {                     // the stage was last read by pair kp - kSt
                const int pp = kp - kSt;
                if (!wait_or_fail(P, &P.done[pp & (kDone - 1)], (pp / kDone) & 1)) return false;
                tc_fence_after();
            }
            tmem_st32(a_lane + s * 64, o);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&P.a_full[s]);
            return true;
        };
        [[maybe_unused]] uint4 corr[8];      // Q4_K: the constant terms of the current 8-block chunk (indexed by kb: local memory)
        // The same in two halves of 32 K-values: the first half's tensor-memory store is under way while the second half
        // is expanded (the store, its wait and the hand-off were a serial tail of every pair).
        auto acquire = [&](int kp) -> bool {
            if (kp >= kSt) {
                const int pp = kp - kSt;
                if (!wait_or_fail(P, &P.done[pp & (kDone - 1)], (pp / kDone) & 1)) return false;
                tc_fence_after();
            }
            return true;
        };
        auto st_half = [&](int kp, int h, const uint32_t* o16) {
            tmem_st16(a_lane + (kp % kSt) * 64 + 16 * h, *(const uint32_t(*)[16]) o16);
        };
        auto release = [&](int kp) {
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&P.a_full[kp % kSt]);
        };
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const int u = kb * 4 + slab, slot = u % NU;
            if (!wait_or_fail(P, &P.raw_full[slot], (u / NU) & 1)) { ok = false; break; }
            const uint8_t* rrow = rbase + (size_t) slot * kUnitBytes<T>;
            uint32_t o[32];
            if constexpr (kIq<T>) {
                constexpr int NWD = kWin<T> / 4;
                uint32_t wv[NWD];
#pragma unroll
                for (int i = 0; i < NWD / 4; ++i) {
                    const uint4 v = *(const uint4*) (rrow + 16 * i);
                    wv[4 * i] = v.x; wv[4 * i + 1] = v.y; wv[4 * i + 2] = v.z; wv[4 * i + 3] = v.w;
                }
                const uint4* sgn = (const uint4*) (smem + kTabOff<T> + kGridBytes<T>);
                // the block's offset in its window, (kb * block bytes) % 16, has period 8 in kb: 8 unrolled variants
#define MAYA_IQ_PAIRS(OFF)                                                                                          \
    if constexpr (T == MAYA_IQ2_S) {                                                                               \
        const uint4* grid = (const uint4*) (smem + kTabOff<T>);                                                    \
        if (team == 0) { iq2s_pair<OFF, 0>(wv, grid, sgn, o); ok = put(kb * 4 + 0, o);                             \
                         if (ok) { iq2s_pair<OFF, 2>(wv, grid, sgn, o); ok = put(kb * 4 + 2, o); } }              \
        else { iq2s_pair<OFF, 1>(wv, grid, sgn, o); ok = put(kb * 4 + 1, o);                                       \
               if (ok) { iq2s_pair<OFF, 3>(wv, grid, sgn, o); ok = put(kb * 4 + 3, o); } }                        \
    } else {                                                                                                       \
        const uint2* grid = (const uint2*) (smem + kTabOff<T>);                                                    \
        if (team == 0) { iq3s_pair<OFF, 0>(wv, grid, sgn, o); ok = put(kb * 4 + 0, o);                             \
                         if (ok) { iq3s_pair<OFF, 2>(wv, grid, sgn, o); ok = put(kb * 4 + 2, o); } }              \
        else { iq3s_pair<OFF, 1>(wv, grid, sgn, o); ok = put(kb * 4 + 1, o);                                       \
               if (ok) { iq3s_pair<OFF, 3>(wv, grid, sgn, o); ok = put(kb * 4 + 3, o); } }                        \
    }
                switch ((kb * kBlkBytes<T>) & 15) {
                    case 0: MAYA_IQ_PAIRS(0) break;
                    case 2: MAYA_IQ_PAIRS(2) break;
                    case 4: MAYA_IQ_PAIRS(4) break;
                    case 6: MAYA_IQ_PAIRS(6) break;
                    case 8: MAYA_IQ_PAIRS(8) break;
                    case 10: MAYA_IQ_PAIRS(10) break;
                    case 12: MAYA_IQ_PAIRS(12) break;
                    default: MAYA_IQ_PAIRS(14) break;
                }
#undef MAYA_IQ_PAIRS
            } else if constexpr (T == MAYA_Q4_K) {
                Q4Scales S;
                q4k_scales(*(const uint4*) rrow, S);
                const int chunk = kb >> 3;           // the team that owns the chunk's correction pair keeps the constant terms
                if ((chunk & 1) == team)
                    corr[kb & 7] = make_uint4(h2_bits(__lows2half2(S.nml[0], S.nml[1])), h2_bits(__lows2half2(S.nml[2], S.nml[3])),
                                              h2_bits(__lows2half2(S.nml[4], S.nml[5])), h2_bits(__lows2half2(S.nml[6], S.nml[7])));
#pragma unroll
                for (int i = 0; i < 2; ++i) {        // the 64 values of quant pair p: low nibbles, then high nibbles
                    const int p = 2 * i + team;
                    const uint4 qa = *(const uint4*) (rrow + 16 + 32 * p), qb = *(const uint4*) (rrow + 32 + 32 * p);
                    const int kp = kb * 4 + chunk + p, sb0 = 4 * i + 2 * team;
                    q4k_stage(qa, qb, 0, S.dl[sb0], S.nml[sb0], o);
                    if (!acquire(kp)) { ok = false; break; }
                    st_half(kp, 0, o);
                    q4k_stage(qa, qb, 1, S.dl[sb0 + 1], S.nml[sb0 + 1], o + 16);
                    st_half(kp, 1, o + 16);
                    release(kp);
                }
                if (ok && (chunk & 1) == team && ((kb & 7) == 7 || kb == nkb - 1)) {      // the chunk's correction pair
#pragma unroll
                    for (int b = 0; b < 8; ++b) {
                        const uint4 c = b <= (kb & 7) ? corr[b] : make_uint4(0u, 0u, 0u, 0u);
                        o[4 * b] = c.x; o[4 * b + 1] = c.y; o[4 * b + 2] = c.z; o[4 * b + 3] = c.w;
                    }
                    ok = put(kb * 4 + chunk + 4, o);
                }
            } else {
#define MAYA_Q80_PAIR(PP)                                                                      \
    if (ok) {                                                                                  \
        q80_stage<2 * (PP)>(rrow, o);                                                          \
        ok = acquire(kb * 4 + (PP));                                                           \
        if (ok) {                                                                              \
            st_half(kb * 4 + (PP), 0, o);                                                      \
            q80_stage<2 * (PP) + 1>(rrow, o + 16);                                             \
            st_half(kb * 4 + (PP), 1, o + 16);                                                 \
            release(kb * 4 + (PP));                                                            \
        }                                                                                      \
    }
                if (team == 0) { MAYA_Q80_PAIR(0) MAYA_Q80_PAIR(2) }
                else { MAYA_Q80_PAIR(1) MAYA_Q80_PAIR(3) }
#undef MAYA_Q80_PAIR
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(&P.raw_empty[slot]);      // 4 warps read a unit; after the 4th it may be overwritten
        }
        // ------------------------------------------------------------ epilogue
        if (ok && !wait_or_fail(P, &P.final, 0)) ok = false;
        tc_fence_after();
        named_bar_sync(3, kDqWarps * 32);            // every expansion warp gets here (all waits are bounded) ...
        ok = !failed(P);                             // ... and they agree: the epilogue's barriers need all of them
        if (tid == 0) MAYA_STAMP(4);                 // accumulators complete, expanding warps met
        if (ok) {
            // The tile leaves through shared memory (both rings are free now: every load was consumed): the warps drop
            // their lanes' values into [activation row][weight row] order, then one bulk copy per activation row
            // writes it out.
            const int q = warp & 3, hs = warp >> 2;                      // hs = 0..3
            const uint32_t lane_base = tmem + ((uint32_t) (32 * q) << 16);
            uint8_t* const stg = smem;
            constexpr int kThreadsEpi = kDqWarps * 32;
            if constexpr (GLU) {
                // Two passes.  First the tile goes from tensor memory to shared memory as h = SwiGLU(gate, up) in f32,
                // [activation row][128]: 16 warps = 4 lane quadrants x 4 groups, a group takes every 4th chunk of 8
                // activation rows.  Then, for the f16 image, every thread rounds 8 consecutive values of a row at a time
                // (4 threads a 32-value group, as maya_mmq_quantize does: the same function, the same bytes) - the
                // groups' amax and sums cost two shuffles each instead of a warp-wide reduction per value.
                __half* b16 = (__half*) stg;                             // [rows][128] f16 image of h
                float* b32 = (float*) (stg + TN * 128 * 2);              // [rows][128] h
                __half* bxa = (__half*) (stg + TN * 128 * 6);            // [rows][4] sum corrections of the row's four 32-value groups
                const int nchunk = (nrows + 7) >> 3;
                const int mcol = 32 * q + lane;
                for (int c = hs; c < nchunk; c += 4) {
                    const int col0 = 8 * c;
                    float v[8], up[8];
                    tmem_ld8(lane_base + col0, v);
                    tmem_ld8(lane_base + kAccCols + col0, up);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (col0 + j < nrows) b32[(col0 + j) * 128 + mcol] = swiglu(v[j], up[j], A.limit);   // uniform in the warp
                }
                if (tid == 0) MAYA_STAMP(5);             // SwiGLU tile in shared memory
                if (A.xq_out) {
                    named_bar_sync(2, kThreadsEpi);
                    const int ch = tid & 15;                             // the row's 8-value chunk; a warp covers two rows
                    for (int r0 = 0; r0 < nrows; r0 += kThreadsEpi / 16) {
                        const int r = r0 + (tid >> 4);
                        const bool live = r < nrows;                     // the same for a group's four threads
                        const float* src = b32 + (live ? r : 0) * 128 + 8 * ch;
                        const float4 lo = *(const float4*) src, hi = *(const float4*) (src + 4);
                        const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                        uint32_t o[4];
                        const __half xa = q8_1_round8(v, o);
                        if (live) {
                            *(uint4*) (b16 + r * 128 + 8 * ch) = make_uint4(o[0], o[1], o[2], o[3]);
                            if ((ch & 3) == 0) bxa[r * 4 + (ch >> 2)] = xa;
                        }
                    }
                }
                if (tid == 0) MAYA_STAMP(6);             // tile rounded
                fence_proxy_async();
                named_bar_sync(1, kThreadsEpi);
                if (tid < nrows) {                                       // one activation row each
                    const int64_t row_g = row0 + tid;
                    if (A.xq_out) {
                        const int64_t ldq = xq_ld(A.w_rows);
                        bulk_store(A.xq_out + row_g * ldq + m0, b16 + tid * 128, 128 * 2);
                        *(uint2*) (A.xq_out + row_g * ldq + A.w_rows + (m0 >> 5)) = *(const uint2*) (bxa + tid * 4);
                        if (blockIdx.x == 0)                             // the zero padding behind the row's corrections
                            for (int64_t c = A.w_rows + A.w_rows / 32; c < ldq; ++c) A.xq_out[row_g * ldq + c] = __float2half_rn(0.0f);
                    }
                    if (A.dst) bulk_store(A.dst + (int64_t) (A.ids ? A.ids[row_g] : row_g) * A.ld_dst + m0, b32 + tid * 128, 128 * 4);
                    bulk_commit();
                }
            } else {
                // 16 warps = 4 lane quadrants x 2 accumulators x 2 groups that take alternate chunks of 16 activation rows
                const int acc = hs & 1, grp = hs >> 1;
                const bool have = m0 + 128 * acc < A.w_rows;             // this warp's accumulator exists
                const uint32_t row_bytes_out = (uint32_t) min(TM, A.w_rows - m0) * 4;
                float* buf = (float*) stg;                               // [rows][256] f32
                const int nchunk = (nrows + 15) >> 4;
                const int mcol = 128 * acc + 32 * q + lane;
                if (have) {
                    for (int c = grp; c < nchunk; c += 2) {
                        const int col0 = 16 * c;
                        float v[16];
                        tmem_ld16(lane_base + acc * kAccCols + col0, v);
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (col0 + j < nrows) buf[(col0 + j) * TM + mcol] = v[j];
                    }
                }
                fence_proxy_async();
                named_bar_sync(1, kThreadsEpi);
                if (tid < nrows) {
                    const int row_g = row0 + tid;
                    bulk_store(A.dst + (int64_t) (A.ids ? A.ids[row_g] : row_g) * A.ld_dst + m0, buf + tid * TM, row_bytes_out);
                    bulk_commit();
                }
            }
            if (tid < nrows) bulk_wait_read<0>();                        // the copies have read shared memory: the block may end
        }
    } else if (warp == kDqWarps) {
        // ------------------------------------------------------------ raw weight units (one lane)
        if (lane == 0) {
            int issued = 0;
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                for (int sl = 0; sl < 4; ++sl) {
                    const int u = kb * 4 + sl, slot = u % NU;
                    if (u >= NU && !wait_or_fail(P, &P.raw_empty[slot], ((u / NU) - 1) & 1)) { ok = false; break; }
                    const int wrow = GLU ? (sl < 2 ? m0 + 64 * sl : A.w_rows + m0 + 64 * (sl - 2)) : m0 + 64 * sl;
                    mbar_expect_tx(&P.raw_full[slot], kUnitBytes<T>);
                    // x: the block's 32-bit words (k-quants), or the 16-byte aligned byte offset of the window around the
                    // i-quant block (the box is then 112 / 144 bytes of each row; past the row's end it reads as zeros)
                    const int x0 = kIq<T> ? (int) (((size_t) kb * kBlkBytes<T>) & ~(size_t) 15) : kb * (kRawRow<T> / 4);
                    tma_load_3d(raw + (size_t) slot * kUnitBytes<T>, &tm_w, &P.raw_full[slot], x0, wrow, found_e);
                    issued = u + 1;
                }
            }
            if (!ok)                                             // let the copies in flight land before the block ends
                for (int u = max(0, issued - NU); u < issued; ++u) wait_or_fail(P, &P.raw_full[u % NU], (u / NU) & 1);
        }
    } else if (warp == kDqWarps + 1 || warp == kDqWarps + 3) {
        // ------------------------------------------------------------ tensor-core issue (one lane of two warps: one
        //                                                              accumulator each, on different schedulers)
        if (lane == 0) {
            const int my = warp == kDqWarps + 1 ? 0 : 1;
            // One product of N = rows rounded up to 16 per accumulator and K = 16: an M = 128 product occupies the
            // tensor core for N / 2 cycles, but only if this thread can issue one that often - a single thread's
            // instruction stream is the limit, so everything here is precomputed or kept incrementally (no divisions,
            // no descriptor construction, the ready barrier tested once before falling into the bounded wait).
            const int n_mma = max(16, (nrows + 15) & ~15);
            const uint32_t idesc = (1u << 4) | ((uint32_t) (n_mma >> 3) << 17) | ((uint32_t) (128 >> 4) << 24);
            const uint64_t bdesc0 = smem_desc_sw128(smem_u32(smem));
            const uint32_t b_hi = (uint32_t) (bdesc0 >> 32), b_lo0 = (uint32_t) bdesc0, b_lo_end = b_lo0 + NB * (kBStage >> 4);
            const uint32_t a0 = tmem + kACol + my * 32, a_end = a0 + kSt * 64, d0 = tmem + my * kAccCols;
            const uint32_t bfull0 = smem_u32(&P.b_full[0]), afull0 = smem_u32(&P.a_full[0]), done0 = smem_u32(&P.done[0]);
            uint32_t b_lo = b_lo0, at = a0, bfull = bfull0, afull = afull0;   // of the next pair of K steps
            uint32_t ph_a = 0, ph_b = 0, first = 0;  // the barriers' phases; first = 0: the first product overwrites
            const int npairs = nkt / 2 + ntp;
            bool ok = true;
            for (int kp = 0; kp < npairs; ++kp) {
                // everything the products need, before the waits
                const uint64_t hi = (uint64_t) b_hi << 32;
                const uint64_t d0b = hi | b_lo, d1b = hi | (b_lo + 2), d2b = hi | (b_lo + 4), d3b = hi | (b_lo + 6);
                const uint32_t done_bar = done0 + ((kp & (kDone - 1)) << 3);
                const bool rb = mbar_test_wait_addr(bfull, ph_b), ra = mbar_test_wait_addr(afull, ph_a);
                if (!rb && !wait_or_fail(P, &P.b_full[(bfull - bfull0) >> 3], ph_b)) { ok = false; break; }   // not there yet: the bounded wait
                if (!ra && !wait_or_fail(P, &P.a_full[(afull - afull0) >> 3], ph_a)) { ok = false; break; }
                tc_fence_after();
                if (my == 0 && kp == 0) MAYA_STAMP(2);       // the first product
                mma_f16_ts_x4_commit(d0, at, d0b, d1b, d2b, d3b, idesc, first, done_bar);
                first = 1;
                at += 64; afull += 8;
                if (at == a_end) { at = a0; afull = afull0; ph_a ^= 1; }
                b_lo += kBStage >> 4; bfull += 8;
                if (b_lo == b_lo_end) { b_lo = b_lo0; bfull = bfull0; ph_b ^= 1; }
            }
            if (my == 0) MAYA_STAMP(3);                      // the last product issued
            if (ok) mma_commit(&P.final);
        }
    } else if (warp == kDqWarps + 2) {
        // ------------------------------------------------------------ activation tiles (one lane)
        if (lane == 0) {
            int issued = 0;
            bool ok = true;
            const uint32_t tx_bytes = big ? kBStage : kBBox;
            const int nmain = nkt / 2;
            for (int kb2 = 0; kb2 < nmain + ntp; ++kb2) {
                const int sb = kb2 % NB;
                // the pair's 64 K-values in the image: K values in order, and after every 32 pairs (or at the end) the
                // chunk's 64 corrections from the tail behind the row's K values
                int xcol;
                if (ntp == 0) xcol = kb2 * 64;
                else {
                    const int c = kb2 / 33, r = kb2 - c * 33;
                    const bool is_corr = r == 32 || kb2 == nmain + ntp - 1;
                    xcol = is_corr ? A.w_cols + 64 * c : (kb2 - c) * 64;
                }
                if (kb2 >= NB) {                             // the slot was last read by pair kb2 - NB
                    const int pp = kb2 - NB;
                    if (!wait_or_fail(P, &P.done[pp % kDone], (pp / kDone) & 1)) { ok = false; break; }
                }
                uint8_t* bt = smem + (size_t) sb * kBStage;
                mbar_expect_tx(&P.b_full[sb], tx_bytes);
                tma_load_2d(bt, &tm_x, &P.b_full[sb], xcol, row0);
                if (big) tma_load_2d(bt + kBBox, &tm_x32, &P.b_full[sb], xcol, row0 + 128);
                issued = kb2 + 1;
            }
            if (!ok)
                for (int kb2 = max(0, issued - NB); kb2 < issued; ++kb2) wait_or_fail(P, &P.b_full[kb2 % NB], (kb2 / NB) & 1);
        }
    }
    if (tid == 0) MAYA_STAMP(7);                    // written back
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
    if (tid == 0 && failed(P) && A.error != nullptr) atomicExch(A.error, 1u);
}

// x rows -> f16 rows of their q8_1 image.  A thread owns 8 consecutive values (one 16-byte store), the 4 threads of a
// 32-value block find its amax with two shuffles.  blockIdx.x is the row, blockIdx.y * 256 + threadIdx.x the 8-value chunk.
// ROUTED = false: image row r is x row ids[r] (ids == nullptr: r).  ROUTED = true: x row t is rounded once and its image
// stored to the k rows pos[t * k + j] (the sorted rows of the token's k routes) - the same bytes as the gathered form
// writes through row_tok, at one eighth of the arithmetic for k = 8.
template<typename X, bool ROUTED>
__global__ void __launch_bounds__(256) mmq_quantize_kernel(const X* __restrict__ x, const int* __restrict__ ids,
                                                           __half* __restrict__ xq, int cols, int64_t ld, int k) {
    const int64_t row = blockIdx.x;
    const int cpr = cols >> 3, c = (int) blockIdx.y * 256 + (int) threadIdx.x;
    const bool live = c < cpr;                       // cpr is a multiple of 4: a block's 4 threads live together
    const int64_t src = (!ROUTED && ids) ? ids[row] : row;
    float v[8];
    if (live) {
        if constexpr (sizeof(X) == 2) {              // bf16 bits, widened exactly
            const uint4 u = *(const uint4*) (x + src * ld + c * 8);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
        } else {
            const float4 a = *(const float4*) (x + src * ld + c * 8), b = *(const float4*) (x + src * ld + c * 8 + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    }
    uint32_t o[4];
    const __half xa = q8_1_round8(v, o);
    // a warp's eight groups: their corrections leave as one 16-byte store when a row is a whole number of warps
    const bool packed = (cols & 255) == 0;
    uint4 cw = make_uint4(0u, 0u, 0u, 0u);
    if (packed) {
        const uint32_t mine = (uint32_t) __half_as_ushort(xa);
        const uint32_t pair = mine | (__shfl_down_sync(0xFFFFFFFFu, mine, 4) << 16);        // lanes 0, 8, 16, 24: groups (2i, 2i + 1)
        const uint32_t p1 = __shfl_sync(0xFFFFFFFFu, pair, 8), p2 = __shfl_sync(0xFFFFFFFFu, pair, 16), p3 = __shfl_sync(0xFFFFFFFFu, pair, 24);
        cw = make_uint4(pair, p1, p2, p3);
    }
    if (!live) return;
    const int64_t ldq = xq_ld(cols);
    const int nd = ROUTED ? k : 1;
    for (int j = 0; j < nd; ++j) {
        const int64_t dr = ROUTED ? (int64_t) ids[row * k + j] : row;
        __half* d = xq + dr * ldq;
        *(uint4*) (d + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
        if (packed) { if ((threadIdx.x & 31) == 0) *(uint4*) (d + cols + (c >> 2)) = cw; }
        else if ((c & 3) == 0) d[cols + (c >> 2)] = xa;
        if (c == 0)                                   // the zero padding behind the row's corrections
            for (int64_t t = cols + cols / 32; t < ldq; ++t) d[t] = __float2half_rn(0.0f);
    }
}

template<typename X>
int launch_quantize(const X* x, const int32_t* ids, void* xq, int type, int64_t cols, int64_t ld, int64_t rows, int k, void* stream) {
    if (!maya_mmq_supported(type)) return refuse(MAYA_ERR_TYPE);
    if (rows <= 0) return MAYA_OK;
    if (!x || !xq || cols <= 0 || cols % 32 || ld < cols || cols > 0x7FFFFFF0ll) return refuse(MAYA_ERR_ARG);
    if (k < 0 || (k > 0 && !ids)) return refuse(MAYA_ERR_ARG);
    if (!aligned16(x) || !aligned16(xq) || (ld * sizeof(X)) % 16) return refuse(MAYA_ERR_ARG);   // 16-byte loads and stores
    const int64_t by = (cols / 8 + 255) / 256;
    if (rows > 0x7FFFFFFFll || by > 65535) return refuse(MAYA_ERR_LIMIT);
    const dim3 grid((unsigned) rows, (unsigned) by);
    if (k > 0) mmq_quantize_kernel<X, true><<<grid, 256, 0, as_stream(stream)>>>(x, ids, (__half*) xq, (int) cols, ld, k);
    else mmq_quantize_kernel<X, false><<<grid, 256, 0, as_stream(stream)>>>(x, ids, (__half*) xq, (int) cols, ld, 0);
    return note_launch(k > 0 ? "mmq_quantize_routed" : "mmq_quantize");
}

// ---- tensor maps (driver entry point looked up once; the library does not link libcuda)
PFN_cuTensorMapEncodeTiled encode_fn() {
    static PFN_cuTensorMapEncodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (PFN_cuTensorMapEncodeTiled) p;
    }();
    return fn;
}
bool make_map(CUtensorMap* m, CUtensorMapDataType dt, int rank, const void* base, const cuuint64_t* dim, const cuuint64_t* stride,
              const cuuint32_t* box, CUtensorMapSwizzle swizzle) {
    PFN_cuTensorMapEncodeTiled fn = encode_fn();
    if (!fn) return false;
    const cuuint32_t es[3] = {1, 1, 1};
    return fn(m, dt, (cuuint32_t) rank, const_cast<void*>(base), dim, stride, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template<int T, bool GLU>
int launch_mmq(const maya_mmq_product* p, const MmqArgs& A, cudaStream_t s) {
    const int64_t mat_rows = p->w_rows, K = p->w_cols;
    const size_t rbw = row_bytes(T, K);
    CUtensorMap tw, tx, tx32;
    std::memset(&tw, 0, sizeof(tw));
    if constexpr (!kIq<T>) {   // weights as 32-bit words: (word in row, row in matrix, matrix); a box = 256 K-values of 64 rows
        const cuuint64_t dim[3] = {(cuuint64_t) (rbw / 4), (cuuint64_t) mat_rows, (cuuint64_t) p->n};
        const cuuint64_t st[2] = {(cuuint64_t) rbw, (cuuint64_t) p->expert_bytes};
        const cuuint32_t box[3] = {(cuuint32_t) (kRawRow<T> / 4), kUnitRows, 1};
        if (!make_map(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, p->w, dim, st, box, CU_TENSOR_MAP_SWIZZLE_NONE))
            return note_launch("mmq weight tensor map");
    } else {                   // i-quants as bytes: a box = the 112 / 144 bytes of 64 rows that hold the block's window;
                               // a row is a multiple of 16 bytes (K a multiple of 2048) and so is every window's start
        const cuuint64_t dim[3] = {(cuuint64_t) rbw, (cuuint64_t) mat_rows, (cuuint64_t) p->n};
        const cuuint64_t st[2] = {(cuuint64_t) rbw, (cuuint64_t) p->expert_bytes};
        const cuuint32_t box[3] = {(cuuint32_t) kRawRow<T>, kUnitRows, 1};
        if (!make_map(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, p->w, dim, st, box, CU_TENSOR_MAP_SWIZZLE_NONE))
            return note_launch("mmq weight tensor map");
    }
    {   // activations: f16 [row][K + tail] (xq_ld); a box = 64 K-values (128 bytes) of 128 or 32 rows, written with the 128-byte swizzle
        const cuuint64_t dim[2] = {(cuuint64_t) xq_ld(K), (cuuint64_t) p->total_rows};
        const cuuint64_t st[1] = {(cuuint64_t) xq_ld(K) * 2};
        const cuuint32_t box[2] = {64, 128}, box32[2] = {64, 32};
        if (!make_map(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p->xq, dim, st, box, CU_TENSOR_MAP_SWIZZLE_128B) ||
            !make_map(&tx32, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p->xq, dim, st, box32, CU_TENSOR_MAP_SWIZZLE_128B))
            return note_launch("mmq activation tensor map");
    }
    constexpr size_t smem = kSmemBytes<T>;
    if (cudaFuncSetAttribute(mmq_kernel<T, GLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess)
        return note_launch("mmq smem attribute");
    const int64_t groups = p->total_rows / TN + p->n;   // an upper bound of sum(ceil(rows_e / 160)), known without the counts
    if (groups > 65535) return refuse(MAYA_ERR_LIMIT);
    const int slab = GLU ? 128 : TM;
    const dim3 grid((unsigned) ((A.w_rows + slab - 1) / slab), (unsigned) groups);
    mmq_kernel<T, GLU><<<grid, kMmqThreads, smem, s>>>(tw, tx, tx32, A);
    return note_launch("mmq");
}

int run_product(const maya_mmq_product* p, bool glu, float limit, cudaStream_t s) {
    if (!p || !p->w || !p->xq || !p->bounds) return refuse(MAYA_ERR_ARG);
    if (!p->dst && !(glu && p->xq_out)) return refuse(MAYA_ERR_ARG);
    if (!maya_mmq_supported(p->type)) return refuse(MAYA_ERR_TYPE);
    if ((p->type == MAYA_IQ2_S || p->type == MAYA_IQ3_S) && p->w_cols % 2048) return refuse(MAYA_ERR_ARG);   // 16-byte aligned rows
    if (p->n <= 0 || p->total_rows <= 0) return MAYA_OK;
    const int64_t out_rows = glu ? p->w_rows / 2 : p->w_rows;
    if (p->w_cols <= 0 || p->w_cols % 256 || out_rows <= 0 || out_rows % 128 || (glu && p->w_rows % 2)) return refuse(MAYA_ERR_ARG);
    if (p->expert_bytes % (size_t) type_bytes(p->type) || p->expert_bytes % 16 || (p->dst && p->ld_dst < out_rows)) {
        std::fprintf(stderr, "maya_mmq_run: expert_bytes %zu is not a whole number of blocks and of 16 bytes, or ld_dst too small\n",
                     p->expert_bytes);
        return refuse(MAYA_ERR_ARG);
    }
    if (!aligned16(p->w) || !aligned16(p->xq) || (p->xq_out && !aligned16(p->xq_out))) return refuse(MAYA_ERR_ARG);
    if (p->dst && (!aligned16(p->dst) || p->ld_dst % 4)) return refuse(MAYA_ERR_ARG);      // rows leave as 16-byte aligned bulk copies
    MmqArgs A{};
    A.w = (const uint8_t*) p->w; A.expert_bytes = p->expert_bytes; A.mat_rows = (int) p->w_rows;
    A.w_rows = (int) out_rows; A.w_cols = (int) p->w_cols; A.n = p->n; A.expert_map = p->expert_map; A.bounds = p->bounds;
    A.ids = p->ids; A.dst = p->dst; A.ld_dst = p->ld_dst; A.xq_out = glu ? (__half*) p->xq_out : nullptr; A.limit = limit;
    A.error = p->error;
    switch (p->type) {
        case MAYA_Q4_K: return glu ? launch_mmq<MAYA_Q4_K, true>(p, A, s) : launch_mmq<MAYA_Q4_K, false>(p, A, s);
        case MAYA_Q8_0: return glu ? launch_mmq<MAYA_Q8_0, true>(p, A, s) : launch_mmq<MAYA_Q8_0, false>(p, A, s);
        case MAYA_IQ2_S: return glu ? launch_mmq<MAYA_IQ2_S, true>(p, A, s) : launch_mmq<MAYA_IQ2_S, false>(p, A, s);
        default: return glu ? launch_mmq<MAYA_IQ3_S, true>(p, A, s) : launch_mmq<MAYA_IQ3_S, false>(p, A, s);
    }
}

}  // namespace
}  // namespace maya

using namespace maya;

#ifdef MAYA_MMQ_STAMPS
// 4 x 4096 x 16 int64: [Q8_0/IQ2_S down, gate/up, Q4_K/IQ3_S down, gate/up][tile][stamp]; slots 14, 15 = rows, K-step pairs
extern "C" __attribute__((visibility("default"))) int maya_mmq_stamps_read(long long* host) {
    return (int) cudaMemcpyFromSymbol(host, g_stamps, sizeof(g_stamps));
}
#endif
extern "C" int maya_mmq_supported(int type) {
    return type == MAYA_Q4_K || type == MAYA_Q8_0 || type == MAYA_IQ2_S || type == MAYA_IQ3_S;
}
extern "C" size_t maya_mmq_q8_bytes(int64_t rows, int64_t cols) {
    if (rows <= 0 || cols <= 0 || cols % 32) return 0;
    return (size_t) rows * (size_t) xq_ld(cols) * sizeof(__half);
}
extern "C" int maya_mmq_quantize(const float* x, const int32_t* ids, void* xq, int type, int64_t cols, int64_t ld,
                                 int64_t rows, void* stream) {
    return launch_quantize<float>(x, ids, xq, type, cols, ld, rows, 0, stream);
}
extern "C" int maya_mmq_quantize_bf16(const uint16_t* x, const int32_t* ids, void* xq, int type, int64_t cols, int64_t ld,
                                      int64_t rows, void* stream) {
    return launch_quantize<uint16_t>(x, ids, xq, type, cols, ld, rows, 0, stream);
}
extern "C" int maya_mmq_quantize_routed(const float* x, const int32_t* pos, int k, void* xq, int type, int64_t cols, int64_t ld,
                                        int64_t tokens, void* stream) {
    if (k <= 0) return refuse(MAYA_ERR_ARG);
    return launch_quantize<float>(x, pos, xq, type, cols, ld, tokens, k, stream);
}
extern "C" int maya_mmq_quantize_routed_bf16(const uint16_t* x, const int32_t* pos, int k, void* xq, int type, int64_t cols,
                                             int64_t ld, int64_t tokens, void* stream) {
    if (k <= 0) return refuse(MAYA_ERR_ARG);
    return launch_quantize<uint16_t>(x, pos, xq, type, cols, ld, tokens, k, stream);
}
extern "C" int maya_mmq_run(const maya_mmq_product* p, void* stream) { return run_product(p, false, 0.0f, as_stream(stream)); }
extern "C" int maya_mmq_run_glu(const maya_mmq_product* p, float limit, void* stream) {
    return run_product(p, true, limit, as_stream(stream));
}
