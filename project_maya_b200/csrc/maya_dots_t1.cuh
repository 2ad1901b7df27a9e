// maya_dots_t1.cuh - the single-column (one token) form of the quantized dots, tuned for the integer-ALU and
// shared-memory limits a B200 SM meets before HBM does on the 2-3 bit formats.
//
// Same integers, same FP32 operation order as maya_dots.cuh (a row's result is bit-identical to rows_dot<T, NR, 1>);
// what changes is how the signed codebook words are dotted:
//   * codebooks are REPLICATED in shared memory so that a warp-wide lookup is free of bank conflicts: IQ2_S entries
//     (8 bytes) 16 times, lane l reading copy l & 15 (two lanes of different half-warps per bank pair); IQ3_S entries
//     (4 bytes) 32 times, lane l reading copy l;
//   * signs are not applied to the codebook bytes.  With m the 0x00 / 0xFF byte mask of the negative weights,
//     sum(s g u) = dp4a(g ^ m, u) - dp4a(m, u): one XOR per four weights on the integer pipe, the correction term on
//     the dot-product pipe;
//   * the byte mask comes from the whole sign byte without masking its nibbles: s * 0x80402010 puts bits 0..3 of any
//     8-bit s at bits 31, 23, 15, 7 and s * 0x08040201 does the same for bits 4..7 (no two partial products that can
//     carry into those positions collide); prmt's sign-replicate mode smears them, in reversed byte order (0x89AB).
#pragma once

#include "maya_dots.cuh"

namespace maya {

__device__ __forceinline__ uint32_t byte_of(uint32_t w, int l) { return __byte_perm(w, 0, 0x4440 + l); }
__device__ __forceinline__ uint32_t prmt_sign(uint32_t x) {
    uint32_t m;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(m) : "r"(x), "r"(0u), "r"(0x89ABu));
    return m;
}
// prmt.b32 in its default mode with the selector as given: nibble n < 8 picks byte n of {a, b}; n + 8 gives the top bit
// of that byte replicated (0x00 for a byte below 0x80: how a zero byte is made without a zero operand).
__device__ __forceinline__ uint32_t prmt_raw(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t sign_mask_lo(uint32_t s) { return prmt_sign(s * 0x80402010u); }   // bits 0..3 of s
__device__ __forceinline__ uint32_t sign_mask_hi(uint32_t s) { return prmt_sign(s * 0x08040201u); }   // bits 4..7 of s

template<int T> struct Rep { static constexpr int n = 1; };
template<> struct Rep<MAYA_IQ2_S> { static constexpr int n = 16; };
template<> struct Rep<MAYA_IQ3_S> { static constexpr int n = 32; };
template<int T> constexpr int kRepTabBytes = Fmt<T>::tab_words * 4 * Rep<T>::n;   // 128 KB (IQ2_S), 64 KB (IQ3_S), 0

// Fill the replicated table: entry e's copy c at word (e * n + c) * words_per_entry.  `tid` of `nt` threads.
template<int T> __device__ __forceinline__ void load_tab_rep(uint32_t* s_tab, int tid, int nt) {
    if constexpr (T == MAYA_IQ2_S) {
        uint2* dst = (uint2*) s_tab;
        const uint2* src = (const uint2*) g_iq2s_grid;
        for (int i = tid; i < 1024 * 16; i += nt) dst[i] = src[i >> 4];
    } else if constexpr (T == MAYA_IQ3_S) {
        for (int i = tid; i < 512 * 32; i += nt) s_tab[i] = g_iq3s_grid[i >> 5];
    }
}

// One q8_1 block of the activation in registers.
__device__ __forceinline__ XQ xq_load1(const XCols& x, int kb) { return xq_load(x, 0, kb); }

template<int T> struct Dec1;

template<> struct Dec1<MAYA_Q8_0> {
    static constexpr int cpb = 1, xblk = 1;
    Dec<MAYA_Q8_0> d;
    __device__ __forceinline__ void load(const uint8_t* blk, int c, const uint32_t* tab, int) { d.load(blk, c, tab); }
    __device__ __forceinline__ float dot(const XQ& v, const XQ&) const {
        int s = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) s = __dp4a(d.w[i], v.u[i], s);
        return __fmul_rn(__fmul_rn(d.d, v.d), (float) s);
    }
};

template<> struct Dec1<MAYA_Q4_K> {
    static constexpr int cpb = 4, xblk = 2;
    Dec<MAYA_Q4_K> d;
    __device__ __forceinline__ void load(const uint8_t* blk, int c, const uint32_t* tab, int) { d.load(blk, c, tab); }
    __device__ __forceinline__ float dot(const XQ& a, const XQ& b) const {
        int s0 = 0, s1 = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) { s0 = __dp4a(d.lo[i], a.u[i], s0); s1 = __dp4a(d.hi[i], b.u[i], s1); }
        const float sd = __fadd_rn(__fmul_rn(a.d, (float) (s0 * d.sc0)), __fmul_rn(b.d, (float) (s1 * d.sc1)));
        const float sm = __fadd_rn(__fmul_rn(a.d, (float) (a.isum * d.m0)), __fmul_rn(b.d, (float) (b.isum * d.m1)));
        return __fsub_rn(__fmul_rn(d.d, sd), __fmul_rn(d.dmin, sm));
    }
};

template<> struct Dec1<MAYA_IQ2_S> {
    static constexpr int cpb = 8, xblk = 1;
    uint32_t gx[8], mk[8];   // codebook word ^ mask, mask
    int ls0, ls1;
    float d;
    __device__ __forceinline__ void load(const uint8_t* blk, int c, const uint32_t* tab, int lane) {
        d = ld_f16(blk);
        const uint32_t qs = ld_u32_a2(blk + 2 + 4 * c), sg = ld_u32_a2(blk + 34 + 4 * c);
        const uint32_t qh = blk[66 + c], sc = blk[74 + c];
        ls0 = (int) (sc & 0x0F);
        ls1 = (int) (sc >> 4);
        const uint2* grid = (const uint2*) tab + (lane & 15);
        // byte l of hw = bits 2l, 2l+1 of qh (the entries' high index bits): fields 0 and 2 by one multiply, 1 and 3 by
        // another; the partial products that miss their byte land on bits the mask drops and none of their sums carries
        // into a kept bit.  An entry index is then ONE byte permute: {qs byte l, hw byte l, 0, 0}.
        const uint32_t hw = ((qh & 0x33u) * 0x1001u + (qh & 0xCCu) * 0x40040u) & 0x03030303u;
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const uint32_t idx = prmt_raw(qs, hw, 0xCC00u + ((4 + l) << 4) + l);
            const uint2 g = grid[idx * 16];
            const uint32_t s = byte_of(sg, l);
            mk[2 * l] = sign_mask_lo(s);
            mk[2 * l + 1] = sign_mask_hi(s);
            gx[2 * l] = g.x ^ mk[2 * l];
            gx[2 * l + 1] = g.y ^ mk[2 * l + 1];
        }
    }
    __device__ __forceinline__ float dot(const XQ& v, const XQ&) const {
        int s0 = 0, s1 = 0, c0 = 0, c1 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            s0 = __dp4a((int) gx[i], v.u[i], s0);
            c0 = __dp4a((int) mk[i], v.u[i], c0);
            s1 = __dp4a((int) gx[4 + i], v.u[4 + i], s1);
            c1 = __dp4a((int) mk[4 + i], v.u[4 + i], c1);
        }
        s0 -= c0;
        s1 -= c1;
        const int sumi = (s0 * ls0 + s1 * ls1 + (s0 + s1) / 2) / 4;
        return __fmul_rn(__fmul_rn(d, v.d), (float) sumi);
    }
};

template<> struct Dec1<MAYA_IQ3_S> {
    static constexpr int cpb = 8, xblk = 1;
    uint32_t gx[8], mk[8];
    int mul;
    float d;
    __device__ __forceinline__ void load(const uint8_t* blk, int c, const uint32_t* tab, int lane) {
        d = ld_f16(blk);
        const uint32_t q0 = ld_u32_a2(blk + 2 + 8 * c), q1 = ld_u32_a2(blk + 6 + 8 * c);
        const uint32_t qh = blk[66 + c], sg = ld_u32_a2(blk + 74 + 4 * c);
        mul = 1 + 2 * (int) ((blk[106 + (c >> 1)] >> (4 * (c & 1))) & 0x0F);
        const uint32_t* grid = tab + lane;
#pragma unroll
        for (int l = 0; l < 8; ++l) {
            const uint32_t idx = byte_of(l < 4 ? q0 : q1, l & 3) | (((qh >> l) & 1) << 8);
            const uint32_t s = byte_of(sg, l >> 1);
            mk[l] = (l & 1) ? sign_mask_hi(s) : sign_mask_lo(s);
            gx[l] = grid[idx * 32] ^ mk[l];
        }
    }
    __device__ __forceinline__ float dot(const XQ& v, const XQ&) const {
        int s = 0, c = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) { s = __dp4a((int) gx[i], v.u[i], s); c = __dp4a((int) mk[i], v.u[i], c); }
        s -= c;
        return __fmul_rn(__fmul_rn(d, v.d), (float) (s * mul));
    }
};

// NR rows against the one staged column; out[r] is bit-identical to rows_dot<T, NR, 1>.
template<int T, int NR>
__device__ __forceinline__ void rows_dot1(const uint8_t* const* rows, const XCols& x, int n_in, int lane,
                                          const uint32_t* tab, float (&out)[NR]) {
    using D = Dec1<T>;
    const int ncalls = (n_in / Fmt<T>::qk) * D::cpb;
    float acc[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) acc[r] = 0.0f;
    for (int k = lane; k < ncalls; k += 32) {
        const int kb = k / D::cpb, ci = k - kb * D::cpb;
        const int xb = kb * (Fmt<T>::qk / 32) + ci * D::xblk;
        const XQ a = xq_load1(x, xb);
        XQ b = a;
        if constexpr (D::xblk == 2) b = xq_load1(x, xb + 1);
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            D dec;
            dec.load(rows[r] + (size_t) kb * Fmt<T>::bytes, ci, tab, lane);
            acc[r] = __fadd_rn(acc[r], dec.dot(a, b));
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) out[r] = warp_sum(acc[r]);
}

// Calls a row of n_in values takes (one lane makes one call per pass of rows_dot1's loop).
template<int T>
__device__ __forceinline__ int calls_per_row(int n_in) { return (n_in / Fmt<T>::qk) * Dec1<T>::cpb; }

// Rows SHORTER than a warp's 32 calls (ncalls = 8 or 16: rows of 256 or 512 values, what a width slice of an expert
// leaves of its down rows): 32 / ncalls rows are taken side by side, lane group g = lane / ncalls working on its own
// rows[r] (the caller passes each lane ITS group's row addresses).  out[r] is valid in every lane of the group and is
// bit-identical to rows_dot1's: there the lanes beyond ncalls add zeros in the first steps of the same shuffle tree.
template<int T, int NR>
__device__ __forceinline__ void rows_dot1_short(const uint8_t* const* rows, const XCols& x, int ncalls, int lane,
                                                const uint32_t* tab, float (&out)[NR]) {
    using D = Dec1<T>;
    const int c = lane & (ncalls - 1);
    const int kb = c / D::cpb, ci = c - kb * D::cpb;
    const int xb = kb * (Fmt<T>::qk / 32) + ci * D::xblk;
    const XQ a = xq_load1(x, xb);
    XQ b = a;
    if constexpr (D::xblk == 2) b = xq_load1(x, xb + 1);
    float acc[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        D dec;
        dec.load(rows[r] + (size_t) kb * Fmt<T>::bytes, ci, tab, lane);
        acc[r] = __fadd_rn(0.0f, dec.dot(a, b));
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        float v = acc[r];
        for (int o = ncalls >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        out[r] = v;
    }
}

}  // namespace maya
