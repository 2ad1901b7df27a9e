// maya_stream.cuh - weight rows streamed through shared memory by the TMA engine, one lane per half GGUF block.
//
// Why: on a B200 SM the 2-3 bit formats are limited by integer-pipe issue and by L1/shared-memory wavefronts long
// before HBM.  Reading a block's fields with 2-byte-aligned loads from global memory (one lane per 32-weight sub-block)
// costs ~7 load instructions, their 64-bit address arithmetic and ~10 L1 wavefronts per sub-block.  Here a warp's rows
// are copied into shared memory by `cp.async.bulk` (no load instructions, no L1 wavefronts for the copy) and each lane
// owns half an 82-byte block (4 sub-blocks): it reads its fields as aligned 32-bit words, and every shift and byte
// selector is a compile-time constant because all lanes of a step handle blocks of the same parity (even blocks start
// 4-byte aligned, odd blocks at +2).
//
// A "stage" is 4 rows x 8 blocks (IQ2_S: 4 x 656 bytes, rows 672 bytes apart in shared memory so that the 32 lanes'
// word reads fall in 32 different banks).  Lane = (g << 3) | (j << 1) | hf handles row g, block 2j + p in step p = 0, 1,
// sub-blocks 4 hf .. 4 hf + 3.  Rows must be a whole number of 8-block segments (n_in % 2048 == 0) and 16-byte aligned,
// which holds for every IQ2_S / IQ3_S shape of the benchmark configurations.
//
// The copies are plain (non-multicast) bulk copies from this GPU's own memory.  Every wait on an mbarrier is bounded;
// a wait that runs out sets an error flag and the kernel carries on to its end without touching the data.
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

__device__ __forceinline__ uint32_t lds32(const uint8_t* p) { return *(const uint32_t*) p; }
__device__ __forceinline__ uint32_t hi_lo(uint32_t a, uint32_t b) { return __byte_perm(a, b, 0x5432); }   // bytes 2..5 of a:b

// ---------------------------------------------------------------- activations: 48-byte blocks
// One q8_1 block as {int4 q[2]; float d; int isum; pad}; a group of 8 (one 256-value weight block) is 4 blocks, 16 bytes
// of padding, 4 blocks (400 bytes).  The 8 distinct addresses a step reads (blocks 2j + p, halves hf) then differ by
// odd and even multiples of 16 bytes that are all distinct modulo 128: one wavefront per quarter-warp.
constexpr int kXBlk = 48;
constexpr int kXHalf = 4 * kXBlk + 16;     // bytes from sub-block 0 to sub-block 4 of a weight block
constexpr int kXGroup = 2 * kXHalf - 16;   // 400 bytes per 8 q8_1 blocks
__host__ __device__ inline size_t xaos_off(int b) {
    return (size_t) (b >> 3) * kXGroup + (size_t) ((b >> 2) & 1) * kXHalf + (size_t) (b & 3) * kXBlk;
}
__host__ __device__ inline size_t xaos_bytes(int nblk) { return (size_t) ((nblk + 7) >> 3) * kXGroup + 16; }
__device__ __forceinline__ void xaos_store_warp(float v, uint8_t* xs, int blk, int lane) {
    const float amax = warp_max(fabsf(v));
    const float dd = fminf(__fdiv_rn(amax, 127.0f), 65504.0f);
    const int qi = amax == 0.0f ? 0 : (int) fmaxf(-127.0f, fminf(127.0f, roundf(__fdiv_rn(v, dd))));
    uint8_t* b = xs + xaos_off(blk);
    ((int8_t*) b)[lane] = (int8_t) qi;
    int s = qi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) {
        *(float*) (b + 32) = __half2float(__float2half_rn(dd));
        *(int*) (b + 36) = s;
    }
}
// the same image from a q8_1 block already in global memory
__device__ __forceinline__ void xaos_from_q8_1(const uint8_t* xq, uint8_t* xs, int nblk, int tid, int nt) {
    for (int i = tid; i < nblk * 8; i += nt) {
        const int b = i >> 3, w = i & 7;
        *(int*) (xs + xaos_off(b) + 4 * w) = *(const int*) (xq + (size_t) b * kQ81Bytes + 4 + 4 * w);
    }
    for (int b = tid; b < nblk; b += nt) {
        const uint8_t* src = xq + (size_t) b * kQ81Bytes;
        int s = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) s = __dp4a(*(const int*) (src + 4 + 4 * w), 0x01010101, s);
        *(float*) (xs + xaos_off(b) + 32) = ld_f16(src);
        *(int*) (xs + xaos_off(b) + 36) = s;
    }
}

// ---------------------------------------------------------------- IQ2_S: half a block (128 weights) per lane
// blk: the block's first byte in shared memory (ODD: 2 mod 4, else 0 mod 4); hf: which half; xb: the image of the q8_1
// block that meets the block's first value; tab_lane: the replicated codebook offset by this lane's copy (lane & 15).
// Sub-blocks are added in ascending order with explicitly rounded operations.
template<int ODD>
__device__ __forceinline__ float iq2s_half(const uint8_t* blk, int hf, const uint8_t* xb, const uint2* tab_lane, float acc) {
    const uint8_t* ab = blk - 2 * ODD;            // 4-byte aligned
    const uint8_t* hb = ab + 16 * hf;
    const uint32_t w0 = lds32(ab);
    const float d = __half2float(__ushort_as_half((unsigned short) (ODD ? (w0 >> 16) : (w0 & 0xFFFFu))));
    uint32_t qs[4], sg[4], Q, S;
    if (ODD) {
#pragma unroll
        for (int i = 0; i < 4; ++i) { qs[i] = lds32(hb + 4 + 4 * i); sg[i] = lds32(hb + 36 + 4 * i); }
        Q = lds32(ab + 68 + 4 * hf);
        S = lds32(ab + 76 + 4 * hf);
    } else {
        uint32_t a[5], b[5];
#pragma unroll
        for (int i = 0; i < 5; ++i) { a[i] = lds32(hb + 4 * i); b[i] = lds32(hb + 32 + 4 * i); }
#pragma unroll
        for (int i = 0; i < 4; ++i) { qs[i] = hi_lo(a[i], a[i + 1]); sg[i] = hi_lo(b[i], b[i + 1]); }
        Q = hi_lo(lds32(ab + 64 + 4 * hf), lds32(ab + 68 + 4 * hf));
        S = hi_lo(lds32(ab + 72 + 4 * hf), lds32(ab + 76 + 4 * hf));
    }
    const uint8_t* xh = xb + hf * kXHalf;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t qh = byte_of(Q, c), sc = byte_of(S, c);
        const int4 u0 = *(const int4*) (xh + c * kXBlk), u1 = *(const int4*) (xh + c * kXBlk + 16);
        const float xd = *(const float*) (xh + c * kXBlk + 32);
        const int u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
        int s0 = 0, s1 = 0, c0 = 0, c1 = 0;
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const uint32_t idx = byte_of(qs[c], l) | ((qh << (8 - 2 * l)) & 0x300);
            const uint2 g = tab_lane[idx * 16];
            const uint32_t s = byte_of(sg[c], l);
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
        acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(d, xd), (float) sumi));
    }
    return acc;
}

constexpr int kSegBlocks = 8;                       // blocks of a row per stage
constexpr int kStageRows = 4;                       // rows per stage
constexpr int kIq2sSegBytes = kSegBlocks * 82;      // 656 bytes copied per row
constexpr int kIq2sRowPitch = kIq2sSegBytes + 16;   // 672: row pitch inside a stage (bank spreading)
constexpr int kIq2sStageBytes = kStageRows * kIq2sRowPitch;   // 2688
constexpr int kIq2sStageTx = kStageRows * kIq2sSegBytes;      // bytes a stage's copies deliver

// One staged segment of 4 IQ2_S rows.  xseg: the activation image of the segment's first value.
__device__ __forceinline__ float iq2s_stage(const uint8_t* stage, const uint8_t* xseg, const uint2* tab_lane, int lane,
                                            float acc) {
    const int g = lane >> 3, j = (lane >> 1) & 3, hf = lane & 1;
    const uint8_t* row = stage + g * kIq2sRowPitch;
    acc = iq2s_half<0>(row + (2 * j) * 82, hf, xseg + (size_t) (2 * j) * kXGroup, tab_lane, acc);
    acc = iq2s_half<1>(row + (2 * j + 1) * 82, hf, xseg + (size_t) (2 * j + 1) * kXGroup, tab_lane, acc);
    return acc;
}
// the sum over a row's 8 lanes (valid in every lane of the row)
__device__ __forceinline__ float stage_row_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    return v;
}

}  // namespace maya
