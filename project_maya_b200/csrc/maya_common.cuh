// maya_common.cuh - shared device helpers: GGUF block geometry, packed loads, warp reductions, launch checks.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "maya_moe.h"

namespace maya {

// ---------------------------------------------------------------- launch bookkeeping (host)
int note_launch(const char* what);          // cudaGetLastError -> status; counts failures
int refuse(int status);                     // counts a refused call, returns status
inline cudaStream_t as_stream(void* s) { return (cudaStream_t) s; }
inline bool aligned16(const void* p) { return (((uintptr_t) p) & 15u) == 0; }

// ---------------------------------------------------------------- GGUF block geometry
// Q8_0  34 B/32 : f16 d | i8 q[32]
// Q4_K 144 B/256: f16 d | f16 dmin | u8 scales[12] | u8 qs[128]
// IQ2_S 82 B/256: f16 d | u8 qs[32] | u8 signs[32] | u8 qh[8] | u8 scales[8]
// IQ3_S 110 B/256: f16 d | u8 qs[64] | u8 qh[8] | u8 signs[32] | u8 scales[4]
// Q8_1  36 B/32 : f16 d | f16 sum | i8 q[32]            (activations)
template<int T> struct Fmt;
template<> struct Fmt<MAYA_Q8_0> { static constexpr int qk = 32, bytes = 34, tab_words = 0; };
template<> struct Fmt<MAYA_Q4_K> { static constexpr int qk = 256, bytes = 144, tab_words = 0; };
template<> struct Fmt<MAYA_IQ2_S> { static constexpr int qk = 256, bytes = 82, tab_words = 2048; };
template<> struct Fmt<MAYA_IQ3_S> { static constexpr int qk = 256, bytes = 110, tab_words = 512; };
// Q5_K  176 B/256: f16 d | f16 dmin | u8 scales[12] | u8 qh[32] | u8 qs[128]
// Q6_K  210 B/256: u8 ql[128] | u8 qh[64] | i8 scales[16] | f16 d
// IQ4_XS 136 B/256: f16 d | u16 scales_h | u8 scales_l[4] | u8 qs[128]
// IQ3_XXS 98 B/256: f16 d | u8 qs[64] | u32 scales_and_signs[8]
// IQ2_XXS 66 B/256: f16 d | per 32 values { u8 qs[4] | u32 scale_and_signs }
template<> struct Fmt<MAYA_Q5_K> { static constexpr int qk = 256, bytes = 176, tab_words = 0; };
template<> struct Fmt<MAYA_Q6_K> { static constexpr int qk = 256, bytes = 210, tab_words = 0; };
template<> struct Fmt<MAYA_IQ4_XS> { static constexpr int qk = 256, bytes = 136, tab_words = 0; };
template<> struct Fmt<MAYA_IQ3_XXS> { static constexpr int qk = 256, bytes = 98, tab_words = 256; };
template<> struct Fmt<MAYA_IQ2_XXS> { static constexpr int qk = 256, bytes = 66, tab_words = 512; };
// IQ1_S  50 B/256: f16 d | u8 qs[32] | u16 qh[8]
template<> struct Fmt<MAYA_IQ1_S> { static constexpr int qk = 256, bytes = 50, tab_words = 2048; };

__host__ __device__ inline int type_bytes(int t) {
    switch (t) {
        case MAYA_Q8_0: return 34;
        case MAYA_Q4_K: return 144;
        case MAYA_IQ3_S: return 110;
        case MAYA_IQ2_S: return 82;
        case MAYA_Q5_K: return 176;
        case MAYA_Q6_K: return 210;
        case MAYA_IQ4_XS: return 136;
        case MAYA_IQ3_XXS: return 98;
        case MAYA_IQ2_XXS: return 66;
        case MAYA_IQ1_S: return 50;
        default: return 0;
    }
}
__host__ __device__ inline int type_qk(int t) { return t == MAYA_Q8_0 ? 32 : type_bytes(t) ? 256 : 0; }
// The four types every path covers (fused single-token kernel, prompt-path GEMM, device-side weight synthesis).
__host__ __device__ inline bool type_is_core(int t) { return t == MAYA_Q8_0 || t == MAYA_Q4_K || t == MAYA_IQ3_S || t == MAYA_IQ2_S; }
__host__ __device__ inline size_t row_bytes(int t, int64_t n) { const int q = type_qk(t); return q ? (size_t) (n / q) * (size_t) type_bytes(t) : 0; }

constexpr int kQ81Bytes = 36;

// ---------------------------------------------------------------- packed loads
// Blocks of 34 / 82 / 110 bytes are only 2-byte aligned inside a row: 32-bit fields are read as two 16-bit halves.
__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) { return *(const uint16_t*) p; }
__device__ __forceinline__ uint32_t ld_u32_a2(const uint8_t* p) { return ld_u16(p) | (ld_u16(p + 2) << 16); }
__device__ __forceinline__ uint32_t ld_u32(const uint8_t* p) { return *(const uint32_t*) p; }
__device__ __forceinline__ float ld_f16(const uint8_t* p) { return __half2float(__ushort_as_half(*(const uint16_t*) p)); }

// ---------------------------------------------------------------- warp reductions
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// One q8_1 block from 32 values held one per lane: d = min(amax / 127, 65504), q = round(v / d) clamped to +-127,
// stored with the f16 sum of the ORIGINAL values (the reference's q8_1_store_warp, glm_fast.cu:165-174).
__device__ __forceinline__ void q8_1_store_warp(float v, uint8_t* dst, int lane) {
    const float amax = warp_max(fabsf(v));
    const float sum = warp_sum(v);
    const float d = fminf(__fdiv_rn(amax, 127.0f), 65504.0f);
    const int q = amax == 0.0f ? 0 : (int) fmaxf(-127.0f, fminf(127.0f, roundf(__fdiv_rn(v, d))));
    ((int8_t*) dst)[4 + lane] = (int8_t) q;
    if (lane == 0) *(__half2*) dst = __floats2half2_rn(d, fmaxf(-65504.0f, fminf(65504.0f, sum)));
}

// clamped SwiGLU (glm_fast.cu:4908-4913); limit = +inf gives silu(g) * u.
__device__ __forceinline__ float swiglu(float g, float u, float limit) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return __fdiv_rn(g, 1.0f + expf(-g)) * u;
}

}  // namespace maya
