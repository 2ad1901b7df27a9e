// maya_dots.cuh - the quantized dot products: GGUF weight blocks (Q8_0, Q4_K, IQ2_S, IQ3_S; Q5_K, Q6_K, IQ4_XS, IQ3_XXS,
// IQ2_XXS, IQ1_S) against q8_1 activations.
//
// Integer semantics follow llama.cpp's vec_dot_*_q8_1 as the reference transcribes them (per 32-value sub-block:
// exact int8 dot, IQ2_S's (s0*l0 + s1*l1 + (s0+s1)/2)/4 with truncating division, IQ3_S's sum * (1 + 2*scale), Q4_K's
// scale and min terms with the integer sum of the activation quants), so every 32-value partial is the same integer
// the reference computes; only the order of the FP32 additions differs.
//
// Work split: a "call" is the part of a weight block one lane handles at once.
//   Q8_0 : 1 call / block  (32 weights, one q8_1 block)
//   Q4_K : 4 calls / block (64 weights: the low and high nibbles of 32 bytes, two q8_1 blocks)
//   IQ2_S: 8 calls / block (32 weights, one q8_1 block)
//   IQ3_S: 8 calls / block (32 weights, one q8_1 block)
// A call first DECODES the weights into signed int8 words (codebook lookup + sign application), then dots them with
// one or more activation columns, so several tokens reuse one decode and every column's result is bit-identical to
// the single-column result.
#pragma once

#include "maya_common.cuh"

namespace maya {

// ---------------------------------------------------------------- activations in shared memory (structure of arrays)
// q8_1 columns are re-laid out when staged: the 8 quant words of a block contiguous and 16-byte aligned, the scale as
// f32, the integer sum of the quants (Q4_K's min term) precomputed once per token instead of once per weight row.
struct XCols {
    const int4* q;     // [ncols][nblk][2]
    const float* d;    // [ncols][nblk]
    const int* isum;   // [ncols][nblk]
    int nblk;          // q8_1 blocks per column
};
__host__ __device__ inline size_t xcols_bytes(int nblk, int ncols) { return (size_t) ncols * nblk * (32 + 4 + 4); }

// Carve the three arrays out of a 16-byte aligned shared buffer.
__device__ __forceinline__ XCols xcols_carve(uint8_t* smem, int nblk, int ncols, int4** q, float** d, int** isum) {
    *q = (int4*) smem;
    *d = (float*) (smem + (size_t) ncols * nblk * 32);
    *isum = (int*) (smem + (size_t) ncols * nblk * 36);
    XCols x;
    x.q = *q; x.d = *d; x.isum = *isum; x.nblk = nblk;
    return x;
}

// Stage `ncols` q8_1 columns (col_stride bytes apart in global memory) into the SoA form.  All threads of the block.
// SUM_F16: the `isum` slot takes the block's stored f16 sum of the unquantized values (as float bits) instead of the integer
// sum of its quants - what IQ1_S's dot needs (its constant term multiplies that sum) and no other type of a launch reads.
template<bool SUM_F16 = false>
__device__ __forceinline__ void xcols_stage(const uint8_t* xq, size_t col_stride, int nblk, int ncols, int4* q, float* d,
                                            int* isum) {
    const int total = nblk * ncols;
    for (int i = threadIdx.x; i < total * 8; i += blockDim.x) {
        const int b = i >> 3, w = i & 7, c = b / nblk, kb = b - c * nblk;
        ((int*) q)[i] = *(const int*) (xq + (size_t) c * col_stride + (size_t) kb * kQ81Bytes + 4 + 4 * w);
    }
    for (int b = threadIdx.x; b < total; b += blockDim.x) {
        const int c = b / nblk, kb = b - c * nblk;
        const uint8_t* src = xq + (size_t) c * col_stride + (size_t) kb * kQ81Bytes;
        d[b] = ld_f16(src);
        if constexpr (SUM_F16) {
            isum[b] = __float_as_int(ld_f16(src + 2));
        } else {
            int s = 0;
#pragma unroll
            for (int w = 0; w < 8; ++w) s = __dp4a(*(const int*) (src + 4 + 4 * w), 0x01010101, s);
            isum[b] = s;
        }
    }
}

struct XQ {          // one q8_1 block in registers
    int u[8];
    float d;
    int isum;
};
__device__ __forceinline__ XQ xq_load(const XCols& x, int col, int kb) {
    XQ v;
    const int b = col * x.nblk + kb;
    const int4 a = x.q[2 * b], c = x.q[2 * b + 1];
    v.u[0] = a.x; v.u[1] = a.y; v.u[2] = a.z; v.u[3] = a.w;
    v.u[4] = c.x; v.u[5] = c.y; v.u[6] = c.z; v.u[7] = c.w;
    v.d = x.d[b];
    v.isum = x.isum[b];
    return v;
}

// ---------------------------------------------------------------- the planar form of the staged columns
// rows_dot's lanes read consecutive calls, i.e. q8_1 blocks XB apart (XB = the blocks a call of the weight type spans:
// 2 for Q4_K and Q5_K, 1 otherwise).  In the form above a lane's 16-byte reads then start 32 * XB bytes apart and the
// eight lanes of a quarter warp fall on 4 / XB bank groups: 2- and 4-way conflicts on every activation load, which made
// the multi-column kernels wait on the shared-memory pipe.  Here a column is stored as 2 * XB planes of 16-byte pieces -
// plane 2 * (block % XB) + half, piece block / XB - and its scales and sums as XB planes of words, so that consecutive
// lanes read consecutive pieces.  Same sizes and the same per-column offsets as the form above.
template<int XB, bool SUM_F16 = false>
__device__ __forceinline__ void xcols_stage_p(const uint8_t* xq, size_t col_stride, int nblk, int ncols, int4* q, float* d,
                                              int* isum) {
    const int total = nblk * ncols, ni = nblk / XB;
    for (int i = threadIdx.x; i < total * 8; i += blockDim.x) {
        const int b = i >> 3, w = i & 7, c = b / nblk, kb = b - c * nblk;
        const int plane = 2 * (kb % XB) + (w >> 2);
        ((int*) q)[(((size_t) c * 2 * XB + plane) * ni + kb / XB) * 4 + (w & 3)] =
            *(const int*) (xq + (size_t) c * col_stride + (size_t) kb * kQ81Bytes + 4 + 4 * w);
    }
    for (int b = threadIdx.x; b < total; b += blockDim.x) {
        const int c = b / nblk, kb = b - c * nblk;
        const uint8_t* src = xq + (size_t) c * col_stride + (size_t) kb * kQ81Bytes;
        const int at = c * nblk + (kb % XB) * ni + kb / XB;
        d[at] = ld_f16(src);
        if constexpr (SUM_F16) {
            isum[at] = __float_as_int(ld_f16(src + 2));
        } else {
            int s = 0;
#pragma unroll
            for (int w = 0; w < 8; ++w) s = __dp4a(*(const int*) (src + 4 + 4 * w), 0x01010101, s);
            isum[at] = s;
        }
    }
}
template<int XB>
__device__ __forceinline__ XQ xq_load_p(const XCols& x, int col, int kb) {
    XQ v;
    const int ni = x.nblk / XB, j = kb % XB, i = kb / XB;
    const int4* p = x.q + ((size_t) col * 2 * XB + 2 * j) * ni + i;
    const int4 a = p[0], c = p[ni];
    v.u[0] = a.x; v.u[1] = a.y; v.u[2] = a.z; v.u[3] = a.w;
    v.u[4] = c.x; v.u[5] = c.y; v.u[6] = c.z; v.u[7] = c.w;
    const int at = col * x.nblk + j * ni + i;
    v.d = x.d[at];
    v.isum = x.isum[at];
    return v;
}

// ---------------------------------------------------------------- sign masks
// Four sign bits (bit i = weight i negative) -> a word whose byte i is 0xFF when bit i is set.  n * 0x10204080 puts
// bit i at bit 8i+7 (the 16 partial products land on distinct bits, so nothing carries); prmt's sign-replicate mode
// then smears each byte's top bit over the byte.
__device__ __forceinline__ uint32_t sign_mask4(uint32_t nibble) {
    uint32_t m;
    const uint32_t x = nibble * 0x10204080u;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(m) : "r"(x), "r"(0u), "r"(0xBA98u));
    return m;
}
// Negate the bytes of g selected by mask m (0x00 / 0xFF per byte); g's bytes are in 0..127 so no carry crosses bytes.
__device__ __forceinline__ int apply_sign4(uint32_t g, uint32_t m) { return (int) ((g ^ m) + (m & 0x01010101u)); }

// ---------------------------------------------------------------- decoded calls
template<int T> struct Dec;

template<> struct Dec<MAYA_Q8_0> {
    static constexpr int cpb = 1, xblk = 1;
    int w[8];
    float d;
    // A block is 34 bytes at a 2-byte aligned address: 8 aligned 32-bit loads from the word that holds its first byte,
    // the tail as one or two 16-bit loads (never past the block), then one prmt per quant word with a selector that
    // depends on the alignment - instead of 17 two-byte loads.
    __device__ __forceinline__ void load(const uint8_t* blk, int, const uint32_t*) {
        const bool odd = (((uintptr_t) blk) & 2u) != 0;               // the block starts in the upper half of a word
        const uint8_t* base = blk - (odd ? 2 : 0);
        uint32_t W[9];
#pragma unroll
        for (int i = 0; i < 8; ++i) W[i] = ld_u32(base + 4 * i);
        W[8] = ld_u16(base + 32);
        if (odd) W[8] |= ld_u16(base + 34) << 16;
        d = __half2float(__ushort_as_half((unsigned short) (odd ? W[0] >> 16 : W[0] & 0xFFFFu)));
        const uint32_t sel = odd ? 0x7654u : 0x5432u;                  // quant word i = bytes 2.. of W[i] : W[i+1], or W[i+1]
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = (int) __byte_perm(W[i], W[i + 1], sel);
    }
    __device__ __forceinline__ float dot(const XQ& v, const XQ&) const {
        int s = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) s = __dp4a(w[i], v.u[i], s);
        return __fmul_rn(__fmul_rn(d, v.d), (float) s);
    }
};

// The 16-byte header of a Q4_K / Q5_K block (d, dmin as f16, then 12 bytes of packed 6-bit scales and mins), read with
// ONE load - a block starts on a 16-byte boundary, as its quants' loads assume too - and the fields of sub-blocks 2j and
// 2j + 1 taken from registers (j < 2: plain 6-bit fields; j >= 2: 4 low bits + 2 high bits).  Read byte by byte it was
// five to nine loads a call, each touching as many cache lines as the warp has blocks.
__device__ __forceinline__ void kquant_header(const uint8_t* blk, int j, float& d, float& dmin, int& sc0, int& sc1, int& m0,
                                              int& m1) {
    const int4 h = *(const int4*) blk;
    const uint32_t dm = (uint32_t) h.x;
    d = __half2float(__ushort_as_half((uint16_t) (dm & 0xFFFF)));
    dmin = __half2float(__ushort_as_half((uint16_t) (dm >> 16)));
    // with s12 = the 12 scale bytes and jj = j % 2: p1 = s12[2 jj], s12[2 jj + 1]; p2 = s12[2 jj + 4 ..]; p3 = s12[2 jj + 8 ..]
    const int sh = 16 * (j & 1);
    const uint32_t p1 = ((uint32_t) h.y >> sh) & 0xFFFFu, p2 = ((uint32_t) h.z >> sh) & 0xFFFFu, p3 = ((uint32_t) h.w >> sh) & 0xFFFFu;
    if (j < 2) {
        sc0 = (int) (p1 & 63u); m0 = (int) (p2 & 63u);
        sc1 = (int) ((p1 >> 8) & 63u); m1 = (int) ((p2 >> 8) & 63u);
    } else {
        sc0 = (int) ((p3 & 0x0Fu) | (((p1 & 0xFFu) >> 6) << 4)); m0 = (int) (((p3 & 0xFFu) >> 4) | (((p2 & 0xFFu) >> 6) << 4));
        sc1 = (int) (((p3 >> 8) & 0x0Fu) | ((p1 >> 14) << 4)); m1 = (int) ((p3 >> 12) | ((p2 >> 14) << 4));
    }
}

template<> struct Dec<MAYA_Q4_K> {
    static constexpr int cpb = 4, xblk = 2;
    int lo[8], hi[8];
    int sc0, sc1, m0, m1;
    float d, dmin;
    __device__ __forceinline__ void load(const uint8_t* blk, int j, const uint32_t*) {
        kquant_header(blk, j, d, dmin, sc0, sc1, m0, m1);
        const int4* q = (const int4*) (blk + 16 + 32 * j);
        const int4 q0 = q[0], q1 = q[1];
        const int qq[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) { lo[i] = qq[i] & 0x0F0F0F0F; hi[i] = (qq[i] >> 4) & 0x0F0F0F0F; }
    }
    __device__ __forceinline__ float dot(const XQ& a, const XQ& b) const {
        int s0 = 0, s1 = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) { s0 = __dp4a(lo[i], a.u[i], s0); s1 = __dp4a(hi[i], b.u[i], s1); }
        const float sd = __fadd_rn(__fmul_rn(a.d, (float) (s0 * sc0)), __fmul_rn(b.d, (float) (s1 * sc1)));
        const float sm = __fadd_rn(__fmul_rn(a.d, (float) (a.isum * m0)), __fmul_rn(b.d, (float) (b.isum * m1)));
        return __fsub_rn(__fmul_rn(d, sd), __fmul_rn(dmin, sm));
    }
};

template<> struct Dec<MAYA_IQ2_S> {
    static constexpr int cpb = 8, xblk = 1;
    int w[8];
    int ls0, ls1;
    float d;
    __device__ __forceinline__ void load(const uint8_t* blk, int c, const uint32_t* tab) {
        d = ld_f16(blk);
        const uint32_t qs = ld_u32_a2(blk + 2 + 4 * c), sg = ld_u32_a2(blk + 34 + 4 * c);
        const uint32_t qh = blk[66 + c], sc = blk[74 + c];
        ls0 = (int) (sc & 0x0F);
        ls1 = (int) (sc >> 4);
        const uint2* grid = (const uint2*) tab;
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const uint32_t idx = ((qs >> (8 * l)) & 0xFF) | ((qh << (8 - 2 * l)) & 0x300);
            const uint2 g = grid[idx];
            const uint32_t s = (sg >> (8 * l)) & 0xFF;
            w[2 * l] = apply_sign4(g.x, sign_mask4(s & 0x0F));
            w[2 * l + 1] = apply_sign4(g.y, sign_mask4(s >> 4));
        }
    }
    __device__ __forceinline__ float dot(const XQ& v, const XQ&) const {
        int s0 = 0, s1 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) { s0 = __dp4a(w[i], v.u[i], s0); s1 = __dp4a(w[4 + i], v.u[4 + i], s1); }
        const int sumi = (s0 * ls0 + s1 * ls1 + (s0 + s1) / 2) / 4;
        return __fmul_rn(__fmul_rn(d, v.d), (float) sumi);
    }
};

template<> struct Dec<MAYA_IQ3_S> {
    static constexpr int cpb = 8, xblk = 1;
    int w[8];
    int mul;
    float d;
    __device__ __forceinline__ void load(const uint8_t* blk, int c, const uint32_t* tab) {
        d = ld_f16(blk);
        const uint32_t q0 = ld_u32_a2(blk + 2 + 8 * c), q1 = ld_u32_a2(blk + 6 + 8 * c);
        const uint32_t qh = blk[66 + c], sg = ld_u32_a2(blk + 74 + 4 * c);
        mul = 1 + 2 * (int) ((blk[106 + (c >> 1)] >> (4 * (c & 1))) & 0x0F);
#pragma unroll
        for (int l = 0; l < 8; ++l) {
            const uint32_t qb = ((l < 4 ? q0 : q1) >> (8 * (l & 3))) & 0xFF;
            const uint32_t idx = qb | (((qh >> l) & 1) << 8);
            w[l] = apply_sign4(tab[idx], sign_mask4((sg >> (4 * l)) & 0x0F));
        }
    }
    __device__ __forceinline__ float dot(const XQ& v, const XQ&) const {
        int s = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) s = __dp4a(w[i], v.u[i], s);
        return __fmul_rn(__fmul_rn(d, v.d), (float) (s * mul));
    }
};

// Q5_K: Q4_K's layout with a fifth bit per value (qh bit sb of byte l belongs to value l of sub-block sb).
template<> struct Dec<MAYA_Q5_K> {
    static constexpr int cpb = 4, xblk = 2;
    int lo[8], hi[8];
    int sc0, sc1, m0, m1;
    float d, dmin;
    __device__ __forceinline__ void load(const uint8_t* blk, int j, const uint32_t*) {
        kquant_header(blk, j, d, dmin, sc0, sc1, m0, m1);
        const int4* h = (const int4*) (blk + 16);
        const int4* q = (const int4*) (blk + 48 + 32 * j);
        const int4 h0 = h[0], h1 = h[1], q0 = q[0], q1 = q[1];
        const int hh[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
        const int qq[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            lo[i] = (qq[i] & 0x0F0F0F0F) | (((hh[i] >> (2 * j)) & 0x01010101) << 4);
            hi[i] = ((qq[i] >> 4) & 0x0F0F0F0F) | (((hh[i] >> (2 * j + 1)) & 0x01010101) << 4);
        }
    }
    __device__ __forceinline__ float dot(const XQ& a, const XQ& b) const {
        int s0 = 0, s1 = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) { s0 = __dp4a(lo[i], a.u[i], s0); s1 = __dp4a(hi[i], b.u[i], s1); }
        const float sd = __fadd_rn(__fmul_rn(a.d, (float) (s0 * sc0)), __fmul_rn(b.d, (float) (s1 * sc1)));
        const float sm = __fadd_rn(__fmul_rn(a.d, (float) (a.isum * m0)), __fmul_rn(b.d, (float) (b.isum * m1)));
        return __fsub_rn(__fmul_rn(d, sd), __fmul_rn(dmin, sm));
    }
};

// Q6_K: a call = one run of 32 values (run r = 4 h + k of half h: ql bytes [64 h + 32 (k & 1), +32), low nibble for
// k < 2 else high; qh bytes [32 h, +32) bits 2k, 2k + 1; value = 6-bit q - 32), two int8 scales (16 values each).
// Blocks of 210 bytes are only 2-byte aligned.
template<> struct Dec<MAYA_Q6_K> {
    static constexpr int cpb = 8, xblk = 1;
    int w[8];
    int sa, sb;
    float d;
    __device__ __forceinline__ void load(const uint8_t* blk, int r, const uint32_t*) {
        const int h = r >> 2, k = r & 3;
        const uint8_t* ql = blk + 64 * h + 32 * (k & 1);
        const uint8_t* qh = blk + 128 + 32 * h;
        const uint32_t sc = ld_u16(blk + 192 + 8 * h + 2 * k);
        sa = (int) (int8_t) (sc & 0xFF);
        sb = (int) (int8_t) (sc >> 8);
        d = ld_f16(blk + 208);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t l4 = (ld_u32_a2(ql + 4 * i) >> (4 * (k >> 1))) & 0x0F0F0F0Fu;
            const uint32_t h2 = ((ld_u32_a2(qh + 4 * i) >> (2 * k)) & 0x03030303u) << 4;
            // q - 32 per byte, q in 0..63: with bit 7 set no byte borrows, and flipping it back leaves the two's complement
            w[i] = (int) ((((l4 | h2) | 0x80808080u) - 0x20202020u) ^ 0x80808080u);
        }
    }
    __device__ __forceinline__ float dot(const XQ& v, const XQ&) const {
        int s0 = 0, s1 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) { s0 = __dp4a(w[i], v.u[i], s0); s1 = __dp4a(w[4 + i], v.u[4 + i], s1); }
        return __fmul_rn(__fmul_rn(d, v.d), (float) (s0 * sa + s1 * sb));
    }
};

// IQ4_XS: a call = sub-block ib of 32 values: 16 bytes of 4-bit indices into the 16-entry non-linear value table (first
// the 16 low nibbles, then the 16 high ones), one 6-bit scale ls - 32.  The table sits in four registers and a lookup
// of four indices is three byte permutes: the low three index bits select within each half of the table, bit 3 picks
// the half (__byte_perm reads three bits of a selector nibble).
template<> struct Dec<MAYA_IQ4_XS> {
    static constexpr int cpb = 8, xblk = 1;
    int w[8];
    int ls;
    float d;
    __device__ __forceinline__ static uint32_t lut4(uint32_t sel16) {      // four 4-bit indices in bits 0..15 -> four table bytes
        constexpr uint32_t t0 = 0xBFAD9881u, t1 = 0xF6EADDCFu, t2 = 0x26190D01u, t3 = 0x71594535u;   // -127 .. 113, little-endian
        const uint32_t lo = __byte_perm(t0, t1, sel16), hi = __byte_perm(t2, t3, sel16);
        return __byte_perm(lo, hi, 0x3210u | ((sel16 & 0x8888u) >> 1));
    }
    __device__ __forceinline__ void load(const uint8_t* blk, int ib, const uint32_t*) {
        d = ld_f16(blk);
        const uint32_t sh = ld_u16(blk + 2), sl = blk[4 + (ib >> 1)];
        ls = (int) (((sl >> (4 * (ib & 1))) & 0x0F) | (((sh >> (2 * ib)) & 3) << 4)) - 32;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t q = ld_u32_a2(blk + 8 + 16 * ib + 4 * i);       // bytes 4i .. 4i + 3: nibbles (b0 lo, b0 hi, b1 lo, ...)
            const uint32_t a = lut4(q & 0xFFFFu), b = lut4(q >> 16);
            w[i] = (int) __byte_perm(a, b, 0x6420);                        // the four low nibbles' values: values 4i .. 4i + 3
            w[4 + i] = (int) __byte_perm(a, b, 0x7531);                    // the high nibbles': values 16 + 4i ..
        }
    }
    __device__ __forceinline__ float dot(const XQ& v, const XQ&) const {
        int s = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) s = __dp4a(w[i], v.u[i], s);
        return __fmul_rn(__fmul_rn(d, v.d), (float) (s * ls));
    }
};

// The 8 sign bits of 8 values from their 7-bit code: the eighth makes the number of set bits even (ksigns_iq2xs).
__device__ __forceinline__ uint32_t ksign8(uint32_t s7) { return s7 | ((__popc(s7) & 1u) << 7); }

// IQ3_XXS: a call = sub-block ib: 8 codebook indices (4 values each) and one 32-bit word of 4 x 7 sign bits + 4-bit scale.
template<> struct Dec<MAYA_IQ3_XXS> {
    static constexpr int cpb = 8, xblk = 1;
    int w[8];
    int ls;
    float d;
    __device__ __forceinline__ void load(const uint8_t* blk, int c, const uint32_t* tab) {
        d = ld_f16(blk);
        const uint32_t q0 = ld_u32_a2(blk + 2 + 8 * c), q1 = ld_u32_a2(blk + 6 + 8 * c), aux = ld_u32_a2(blk + 66 + 4 * c);
        ls = (int) (aux >> 28);
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const uint32_t s8 = ksign8((aux >> (7 * l)) & 127u);
            const uint32_t qa = ((l < 2 ? q0 : q1) >> (16 * (l & 1))) & 0xFFFFu;
            w[2 * l] = apply_sign4(tab[qa & 0xFF], sign_mask4(s8 & 0x0F));
            w[2 * l + 1] = apply_sign4(tab[qa >> 8], sign_mask4(s8 >> 4));
        }
    }
    __device__ __forceinline__ float dot(const XQ& v, const XQ&) const {
        int s = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) s = __dp4a(w[i], v.u[i], s);
        return __fmul_rn(__fmul_rn(d, v.d), (float) ((ls * s + s / 2) / 2));
    }
};

// IQ2_XXS: a call = sub-block ib: 4 codebook indices (8 values each), then 4 x 7 sign bits + 4-bit scale.
template<> struct Dec<MAYA_IQ2_XXS> {
    static constexpr int cpb = 8, xblk = 1;
    int w[8];
    int ls;
    float d;
    __device__ __forceinline__ void load(const uint8_t* blk, int c, const uint32_t* tab) {
        d = ld_f16(blk);
        const uint32_t qi = ld_u32_a2(blk + 2 + 8 * c), aux = ld_u32_a2(blk + 6 + 8 * c);
        ls = (int) (aux >> 27) | 1;                  // 2 * scale + 1
        const uint2* grid = (const uint2*) tab;
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const uint2 g = grid[(qi >> (8 * l)) & 0xFF];
            const uint32_t s8 = ksign8((aux >> (7 * l)) & 127u);
            w[2 * l] = apply_sign4(g.x, sign_mask4(s8 & 0x0F));
            w[2 * l + 1] = apply_sign4(g.y, sign_mask4(s8 >> 4));
        }
    }
    __device__ __forceinline__ float dot(const XQ& v, const XQ&) const {
        int s = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) s = __dp4a(w[i], v.u[i], s);
        return __fmul_rn(__fmul_rn(d, v.d), (float) (s * ls / 8));
    }
};

// IQ1_S: a call = sub-block ib: four 11-bit codebook indices (8 values in {-1, 0, 1} each, kept as value + 1 in nibbles),
// one 3-bit scale and the sign of the +-1/8 shift.  sum((g + delta) x) = sum((g + 1) q) d8 + (delta - 1) * S with S the
// q8_1 block's stored sum of the unquantized activations (staged into the isum slot: xcols_stage<true>).
template<> struct Dec<MAYA_IQ1_S> {
    static constexpr int cpb = 8, xblk = 1;
    int w[8];
    float d1q, delta;
    __device__ __forceinline__ void load(const uint8_t* blk, int c, const uint32_t* tab) {
        const uint32_t qs = ld_u32_a2(blk + 2 + 4 * c), qh = ld_u16(blk + 34 + 2 * c);
        d1q = ld_f16(blk) * (float) (2 * ((qh >> 12) & 7) + 1);
        delta = (qh & 0x8000u) ? -1.125f : -0.875f;
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const uint32_t g = tab[((qs >> (8 * l)) & 0xFF) | (((qh >> (3 * l)) & 7) << 8)];
            w[2 * l] = (int) (g & 0x0F0F0F0Fu);
            w[2 * l + 1] = (int) ((g >> 4) & 0x0F0F0F0Fu);
        }
    }
    __device__ __forceinline__ float dot(const XQ& v, const XQ&) const {
        int s = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) s = __dp4a(w[i], v.u[i], s);
        return __fmul_rn(d1q, __fadd_rn(__fmul_rn(v.d, (float) s), __fmul_rn(__int_as_float(v.isum), delta)));
    }
};

// ---------------------------------------------------------------- codebooks
// One device copy per translation unit (no relocatable device code needed); generated at build time.
#define MAYA_GRID_QUAL static __device__ const
#define MAYA_IQ2S_GRID g_iq2s_grid
#define MAYA_IQ3S_GRID g_iq3s_grid
#define MAYA_IQ2XXS_GRID g_iq2xxs_grid
#define MAYA_IQ3XXS_GRID g_iq3xxs_grid
#define MAYA_IQ1S_GRID g_iq1s_grid
#include "generated/maya_iq_grids.inc"
#undef MAYA_IQ1S_GRID
#undef MAYA_IQ2S_GRID
#undef MAYA_IQ3S_GRID
#undef MAYA_IQ2XXS_GRID
#undef MAYA_IQ3XXS_GRID
#undef MAYA_GRID_QUAL

template<int T> __device__ __forceinline__ void load_tab(uint32_t* s_tab) {
    if constexpr (Fmt<T>::tab_words > 0) {
        const uint32_t* src = T == MAYA_IQ2_S ? (const uint32_t*) g_iq2s_grid : T == MAYA_IQ3_S ? (const uint32_t*) g_iq3s_grid
                              : T == MAYA_IQ2_XXS ? (const uint32_t*) g_iq2xxs_grid : T == MAYA_IQ1_S ? (const uint32_t*) g_iq1s_grid
                              : (const uint32_t*) g_iq3xxs_grid;
        for (int i = threadIdx.x; i < Fmt<T>::tab_words; i += blockDim.x) s_tab[i] = src[i];
    }
}

// ---------------------------------------------------------------- NR rows x NC columns, one warp
// rows[r]: the row's first block; calls are lane-strided over the row (call c = lane, lane + 32, ...); each lane adds
// its calls in ascending order (explicitly rounded multiplies and adds, never contracted, so a column's bits do not
// depend on how many columns the instantiation carries), then the butterfly sum.  out[r][c].
// x: columns staged by xcols_stage_p<XL> (XL = the call's span in q8_1 blocks unless two types share the columns).
template<int T, int NR, int NC, int XL = Dec<T>::xblk>
__device__ __forceinline__ void rows_dot(const uint8_t* const* rows, const XCols& x, int ncols, int n_in, int lane,
                                         const uint32_t* tab, float (&out)[NR][NC]) {
    using D = Dec<T>;
    const int ncalls = (n_in / Fmt<T>::qk) * D::cpb;
    float acc[NR][NC];
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[r][c] = 0.0f;
    // The decoded rows of a pass stay in registers and a column's activation blocks are read from shared memory ONCE for
    // all of them (the dots were bound by shared-memory wavefronts when every row re-read them);
    // RP rows a pass: all NR, two for the types whose call spans two q8_1 blocks (twice the registers a row).
    constexpr int RP = D::xblk == 2 ? (NR < 2 ? NR : 2) : NR;
    for (int k = lane; k < ncalls; k += 32) {
        const int kb = k / D::cpb, ci = k - kb * D::cpb;
        const int xb = kb * (Fmt<T>::qk / 32) + ci * D::xblk;
#pragma unroll
        for (int r0 = 0; r0 < NR; r0 += RP) {
            D dec[RP];
#pragma unroll
            for (int j = 0; j < RP; ++j)
                if (r0 + j < NR) dec[j].load(rows[r0 + j] + (size_t) kb * Fmt<T>::bytes, ci, tab);
#pragma unroll
            for (int c = 0; c < NC; ++c)
                if (c < ncols) {
                    const XQ a = xq_load_p<XL>(x, c, xb);
                    XQ b = a;
                    if constexpr (D::xblk == 2) b = xq_load_p<XL>(x, c, xb + 1);
#pragma unroll
                    for (int j = 0; j < RP; ++j)
                        if (r0 + j < NR) acc[r0 + j][c] = __fadd_rn(acc[r0 + j][c], dec[j].dot(a, b));
                }
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
        for (int c = 0; c < NC; ++c) out[r][c] = warp_sum(acc[r][c]);
}

}  // namespace maya
