// maya_stream.cuh - weight rows streamed through shared memory by the TMA engine (cp.async.bulk + mbarrier) and the
// single-token dots that read them there.
//
// Why: on a B200 SM the 2-3 bit formats are limited by instruction issue long before HBM.  An integer-pipe
// instruction (logic, shift, byte permute) takes two issue cycles of its scheduler, everything else one, and the
// single-token IQ2_S dot that reads a block's fields from global memory costs ~217 such cycles per 32 weights.  Here
//   * the rows arrive in shared memory without load instructions, address arithmetic or scoreboard stalls
//     (one bulk copy per row segment, completion counted on an mbarrier, a ring of slots per warp);
//   * one lane owns HALF a block (4 sub-blocks), so a block's fields are read as few aligned words and a lane's
//     alignment selector is a constant;
//   * the two high index bits of a sub-block's four codebook entries are spread to byte positions with two multiplies,
//     so that an entry index is ONE byte permute (low byte from qs, high byte from the spread word);
//   * sign bytes, qh and scale bytes are read as bytes (the load/store pipe has room, the integer pipe has none).
//
// Bit-exactness with rows_dot1 (maya_dots_t1.cuh): that routine gives call k (= sub-block k of the row) to lane
// L = k mod 32, adds a lane's calls in ascending k and then sums the lanes with the xor butterfly 16, 8, 4, 2, 1.  Here
// the lanes of a row are (j, hf) = block j mod 4, half hf, and each keeps FOUR accumulators a[i], one per sub-block of
// its half: a[i] is exactly the accumulator of rows_dot1's lane L = 8 j + 4 hf + i, filled in the same order.  The
// butterfly then runs over (j, hf) with shuffles (xor 16, 8 = the bits of j; xor 4 = hf) and over i inside the lane
// (xor 2: a0 + a2, a1 + a3; xor 1: their sum): the same additions in the same order, so the same bits.
//
// The copies are plain (non-multicast) bulk copies from this GPU's own memory.  Every wait on an mbarrier is bounded;
// a wait that runs out returns false and the caller carries on to its end without touching the data.
#pragma once

#include "maya_dots_t1.cuh"

namespace maya {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// global -> this block's shared memory, completion counted in bytes on `bar`.  16-byte aligned, size % 16 == 0.
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// The non-suspending form: one look at the barrier.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait (every lane polls).  false: gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (unsigned i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(32);
    }
    return false;
}
// Order this thread's earlier shared-memory reads/writes before later async-proxy (TMA) writes to the same bytes.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------- activation image: 144 bytes per 128 values
// Four q8_1 blocks as {int q[4][8]; float d[4]}.  The eight lanes of a row read eight consecutive half-block images
// with 16-byte loads: 144 bytes = 36 words apart, i.e. eight different bank quads - one wavefront a load.
constexpr int kXHalfBytes = 144;
__host__ __device__ inline size_t ximg_bytes(int nblk32) { return (size_t) ((nblk32 + 3) / 4) * kXHalfBytes; }
__device__ __forceinline__ uint8_t* ximg_q(uint8_t* img, int blk32) { return img + (size_t) (blk32 >> 2) * kXHalfBytes + (blk32 & 3) * 32; }
__device__ __forceinline__ float* ximg_d(uint8_t* img, int blk32) { return (float*) (img + (size_t) (blk32 >> 2) * kXHalfBytes + 128) + (blk32 & 3); }
// q8_1 of 32 values held one per lane, into block blk32 of the image (the reference's q8_1_store_warp, glm_fast.cu:165-174,
// with the scale kept as the f32 value of the f16 field)
__device__ __forceinline__ void ximg_store_warp(float v, uint8_t* img, int blk32, int lane) {
    const float amax = warp_max(fabsf(v));
    const float dd = fminf(__fdiv_rn(amax, 127.0f), 65504.0f);
    const int qi = amax == 0.0f ? 0 : (int) fmaxf(-127.0f, fminf(127.0f, roundf(__fdiv_rn(v, dd))));
    ((int8_t*) ximg_q(img, blk32))[lane] = (int8_t) qi;
    if (lane == 0) *ximg_d(img, blk32) = __half2float(__float2half_rn(dd));
}
// the same image from q8_1 blocks in global memory (36 bytes each)
__device__ __forceinline__ void ximg_from_q8_1(const uint8_t* xq, uint8_t* img, int nblk32, int tid, int nt) {
    for (int i = tid; i < nblk32 * 8; i += nt) {
        const int b = i >> 3, w = i & 7;
        ((int*) ximg_q(img, b))[w] = *(const int*) (xq + (size_t) b * kQ81Bytes + 4 + 4 * w);
    }
    for (int b = tid; b < nblk32; b += nt) *ximg_d(img, b) = ld_f16(xq + (size_t) b * kQ81Bytes);
}

// ---------------------------------------------------------------- IQ2_S / IQ3_S stages: 4 rows x 8 blocks
template<int T> struct Stage;
template<> struct Stage<MAYA_IQ2_S> {
    static constexpr int rows = 4, seg_vals = 2048;
    static constexpr int seg_bytes = 8 * 82;       // 656 = 41 x 16
    static constexpr int pitch = seg_bytes + 16;   // 672: the four rows' words fall in different bank octets
    static constexpr int bytes = rows * pitch;     // 2688
};
template<> struct Stage<MAYA_IQ3_S> {
    static constexpr int rows = 4, seg_vals = 2048;
    static constexpr int seg_bytes = 8 * 110;      // 880 = 55 x 16
    static constexpr int pitch = seg_bytes + 16;   // 896
    static constexpr int bytes = rows * pitch;     // 3584
};
// Q8_0: 2 rows x 32 blocks (1024 values); 1088 = 8 x 128 + 64 bytes a row, so the second row's words use the banks
// the first row's 8.5-word block stride leaves free.
template<> struct Stage<MAYA_Q8_0> {
    static constexpr int rows = 2, seg_vals = 1024;
    static constexpr int seg_bytes = 32 * 34;      // 1088 = 68 x 16
    static constexpr int pitch = seg_bytes;
    static constexpr int bytes = rows * pitch;     // 2176
};
constexpr int kStageSlotBytes = 3584;              // one ring slot holds a stage of any of the three

// prmt.b32 in its default mode with the selector as given: nibble n < 8 picks byte n of {a, b}; n + 8 gives the top bit
// of that byte replicated (0x00 for a byte below 0x80: how a zero byte is made without a zero operand).
__device__ __forceinline__ uint32_t prmt_raw(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// Half an IQ2_S block (sub-blocks 4 hf .. 4 hf + 3) against its half-block activation image.
//   blk  the block's first byte in shared memory; odd: the block starts 2 bytes past a word boundary (blocks are 82
//        bytes, row segments 16-byte aligned: odd-numbered blocks), a per-lane constant; xh the 144-byte image;
//   tab_lane the replicated codebook offset by this lane's copy.  acc[i] += the product of sub-block 4 hf + i.
template<bool SIGN_BYTES, int REP = 16>
__device__ __forceinline__ void iq2s_half(const uint8_t* blk, int hf, int odd, const uint8_t* xh, const uint2* tab_lane,
                                          float (&acc)[4]) {
    const float d = __half2float(*(const __half*) blk);
    const uint8_t* ab = blk - 2 * odd + 16 * hf;                 // word aligned
    const uint32_t sel = odd ? 0x7654u : 0x5432u;                // field word i = bytes 2..5 of W[i]:W[i+1], or W[i+1]
    uint32_t W[5], qs[4];
#pragma unroll
    for (int i = 0; i < 5; ++i) W[i] = *(const uint32_t*) (ab + 4 * i);
#pragma unroll
    for (int i = 0; i < 4; ++i) qs[i] = __byte_perm(W[i], W[i + 1], sel);
    uint32_t sg[4];
    if constexpr (!SIGN_BYTES) {
        uint32_t V[5];
#pragma unroll
        for (int i = 0; i < 5; ++i) V[i] = *(const uint32_t*) (ab + 32 + 4 * i);
#pragma unroll
        for (int i = 0; i < 4; ++i) sg[i] = __byte_perm(V[i], V[i + 1], sel);
    }
    const uint8_t* sgb = blk + 34 + 16 * hf;
    const uint8_t* qhb = blk + 66 + 4 * hf;
    const uint8_t* scb = blk + 74 + 4 * hf;
    const float4 xd = *(const float4*) (xh + 128);
    const float xds[4] = {xd.x, xd.y, xd.z, xd.w};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t qh = qhb[c], sc = scb[c];
        // byte l of hw = bits 2l, 2l+1 of qh: fields 0 and 2 by one multiply, 1 and 3 by another; the partial products
        // that miss their byte land on bits the mask drops, and none of their sums carries into a kept bit.
        const uint32_t hw = ((qh & 0x33u) * 0x1001u + (qh & 0xCCu) * 0x40040u) & 0x03030303u;
        const int4 u0 = *(const int4*) (xh + 32 * c), u1 = *(const int4*) (xh + 32 * c + 16);
        const int u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
        int s0 = 0, s1 = 0, c0 = 0, c1 = 0;
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const uint32_t idx = prmt_raw(qs[c], hw, 0xCC00u + ((4 + l) << 4) + l);        // {qs byte l, hw byte l, 0, 0}
            const uint2 g = tab_lane[idx * REP];
            const uint32_t s = SIGN_BYTES ? (uint32_t) sgb[4 * c + l] : byte_of(sg[c], l);
            const uint32_t m0 = sign_mask_lo(s), m1 = sign_mask_hi(s);
            if (l < 2) {
                s0 = __dp4a((int) (g.x ^ m0), u[2 * l], s0);
                c0 = __dp4a((int) m0, u[2 * l], c0);
                s0 = __dp4a((int) (g.y ^ m1), u[2 * l + 1], s0);
                c0 = __dp4a((int) m1, u[2 * l + 1], c0);
            } else {
                s1 = __dp4a((int) (g.x ^ m0), u[2 * l], s1);
                c1 = __dp4a((int) m0, u[2 * l], c1);
                s1 = __dp4a((int) (g.y ^ m1), u[2 * l + 1], s1);
                c1 = __dp4a((int) m1, u[2 * l + 1], c1);
            }
        }
        s0 -= c0;
        s1 -= c1;
        const int ls0 = (int) (sc & 0x0F), ls1 = (int) (sc >> 4);
        const int sumi = (s0 * ls0 + s1 * ls1 + (s0 + s1) / 2) / 4;
        acc[c] = __fadd_rn(acc[c], __fmul_rn(__fmul_rn(d, xds[c]), (float) sumi));
    }
}

// One staged segment (8 blocks) of 4 IQ2_S rows: lane (g, j, hf) = (lane >> 3, (lane >> 1) & 3, lane & 1) takes half
// hf of blocks j and j + 4 of row g.  ximg_seg: the activation image at the segment's first value.
template<bool SIGN_BYTES, int REP = 16>
__device__ __forceinline__ void iq2s_stage(const uint8_t* stage, const uint8_t* ximg_seg, const uint2* tab_lane, int lane,
                                           float (&acc)[4]) {
    const int g = lane >> 3, j = (lane >> 1) & 3, hf = lane & 1, odd = j & 1;
    const uint8_t* row = stage + g * Stage<MAYA_IQ2_S>::pitch;
    iq2s_half<SIGN_BYTES, REP>(row + j * 82, hf, odd, ximg_seg + (size_t) (2 * j + hf) * kXHalfBytes, tab_lane, acc);
    iq2s_half<SIGN_BYTES, REP>(row + (j + 4) * 82, hf, odd, ximg_seg + (size_t) (2 * (j + 4) + hf) * kXHalfBytes, tab_lane, acc);
}

// The row sum of the four accumulators of a row's eight lanes, in rows_dot1's butterfly order (valid in all 8 lanes).
__device__ __forceinline__ float iq_row_sum(float (&a)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] += __shfl_xor_sync(0xffffffffu, a[i], 4);     // L ^ 16
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] += __shfl_xor_sync(0xffffffffu, a[i], 2);     // L ^ 8
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] += __shfl_xor_sync(0xffffffffu, a[i], 1);     // L ^ 4
    return (a[0] + a[2]) + (a[1] + a[3]);                                          // L ^ 2, then L ^ 1
}

// ---------------------------------------------------------------- Q8_0 stages: 2 rows x 32 blocks
// Lane (g, l) = (lane >> 4, lane & 15) takes blocks l and l + 16 of the window: rows_dot1's lanes L = l and l + 16.
__device__ __forceinline__ void q8_0_stage(const uint8_t* stage, const uint8_t* ximg_seg, int lane, float (&acc)[2]) {
    const int g = lane >> 4, l = lane & 15;
    const uint8_t* row = stage + g * Stage<MAYA_Q8_0>::pitch;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int b = l + 16 * i;
        Dec<MAYA_Q8_0> dec;
        dec.load(row + b * 34, 0, nullptr);
        const uint8_t* xq = ximg_seg + (size_t) (b >> 2) * kXHalfBytes + (b & 3) * 32;
        const int4 u0 = *(const int4*) xq, u1 = *(const int4*) (xq + 16);
        const float xd = *((const float*) (ximg_seg + (size_t) (b >> 2) * kXHalfBytes + 128) + (b & 3));
        int s = 0;
        s = __dp4a(dec.w[0], u0.x, s); s = __dp4a(dec.w[1], u0.y, s); s = __dp4a(dec.w[2], u0.z, s); s = __dp4a(dec.w[3], u0.w, s);
        s = __dp4a(dec.w[4], u1.x, s); s = __dp4a(dec.w[5], u1.y, s); s = __dp4a(dec.w[6], u1.z, s); s = __dp4a(dec.w[7], u1.w, s);
        acc[i] = __fadd_rn(acc[i], __fmul_rn(__fmul_rn(dec.d, xd), (float) s));
    }
}
// the row sum over a row's sixteen lanes (valid in all of them): xor 16 inside the lane, then 8, 4, 2, 1
__device__ __forceinline__ float q8_0_row_sum(const float (&a)[2]) {
    float v = a[0] + a[1];
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v;
}

}  // namespace maya
