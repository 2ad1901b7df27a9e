// synth.cu - synthetic expert weights for tests and benchmarks: quantizers written from the GGUF block definitions.
//
// The reference quantizes through ggml's quantizers, which are not part of its tree; these are this library's own
// (a different, simpler fit: one scale estimate per sub-block, nearest-codeword search by exhaustion for the
// i-quants).  Any output is a valid block of its type, which is all the kernels' parity depends on; the value
// distribution is that of N(0, sigma) weights rounded to the type's grid.
//
//   maya_quantize_weights_host : host floats -> host blocks (small cases, CPU tests)
//   maya_synth_weights         : device; draws N(0, sigma) from a counter-based generator and quantizes in one pass,
//                                one warp per 256 values (lane l holds values 8l .. 8l+7)
#include <math.h>
#include <string.h>

#include "maya_dots.cuh"

namespace maya {
namespace {

#define MAYA_GRID_QUAL static const
#define MAYA_IQ2S_GRID h_iq2s_grid
#define MAYA_IQ3S_GRID h_iq3s_grid
#include "generated/maya_iq_grids.inc"
#undef MAYA_IQ2S_GRID
#undef MAYA_IQ3S_GRID
#undef MAYA_GRID_QUAL

__host__ __device__ inline unsigned long long iq2s_entry(int i) {
#ifdef __CUDA_ARCH__
    return g_iq2s_grid[i];
#else
    return h_iq2s_grid[i];
#endif
}
__host__ __device__ inline unsigned int iq3s_entry(int i) {
#ifdef __CUDA_ARCH__
    return g_iq3s_grid[i];
#else
    return h_iq3s_grid[i];
#endif
}

// ---------------------------------------------------------------- counter-based normal generator
__host__ __device__ inline uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// value `i` of stream `seed`: Box-Muller over two 24-bit uniforms of one 64-bit hash
__host__ __device__ inline float normal_at(uint64_t seed, uint64_t i) {
    const uint64_t h = mix64(seed * 0xD1342543DE82EF95ull + i);
    const float u1 = ((float) ((h >> 40) & 0xFFFFFF) + 1.0f) * (1.0f / 16777216.0f);
    const float u2 = (float) ((h >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);
    return sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
}

__host__ __device__ inline uint16_t f2h_bits(float f) {
#ifdef __CUDA_ARCH__
    return __half_as_ushort(__float2half_rn(f));
#else
    const __half h = __float2half_rn(f);
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
#endif
}
__host__ __device__ inline float h2f_bits(uint16_t b) {
#ifdef __CUDA_ARCH__
    return __half2float(__ushort_as_half(b));
#else
    __half h;
    memcpy(&h, &b, 2);
    return __half2float(h);
#endif
}
__host__ __device__ inline int iround_clamp(float v, int lo, int hi) {
    const int q = (int) rintf(v);
    return q < lo ? lo : q > hi ? hi : q;
}

// nearest IQ2_S codeword (8 magnitudes from {8, 25, 43}) to a[0..8)
__host__ __device__ inline int nearest_iq2s(const float* a) {
    int best = 0;
    float bd = 3.0e38f;
    for (int e = 0; e < 1024; ++e) {
        const unsigned long long g = iq2s_entry(e);
        float dsum = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float t = a[i] - (float) ((g >> (8 * i)) & 0xFF);
            dsum += t * t;
        }
        if (dsum < bd) { bd = dsum; best = e; }
    }
    return best;
}
// nearest IQ3_S codeword (4 magnitudes from {1, 3, .., 15}) to a[0..4)
__host__ __device__ inline int nearest_iq3s(const float* a) {
    int best = 0;
    float bd = 3.0e38f;
    for (int e = 0; e < 512; ++e) {
        const unsigned int g = iq3s_entry(e);
        float dsum = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float t = a[i] - (float) ((g >> (8 * i)) & 0xFF);
            dsum += t * t;
        }
        if (dsum < bd) { bd = dsum; best = e; }
    }
    return best;
}

// ---------------------------------------------------------------- host quantizers (one block at a time)
void host_q8_0(const float* x, uint8_t* o) {
    float amax = 0.0f;
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(x[i]));
    const uint16_t hd = f2h_bits(amax / 127.0f);
    const float d = h2f_bits(hd), id = d > 0.0f ? 1.0f / d : 0.0f;
    memcpy(o, &hd, 2);
    for (int i = 0; i < 32; ++i) o[2 + i] = (uint8_t) (int8_t) iround_clamp(x[i] * id, -127, 127);
}

void host_q4_K(const float* x, uint8_t* o) {
    float scale[8], mn[8], smax = 0.0f, mmax = 0.0f;
    for (int j = 0; j < 8; ++j) {
        float lo = 0.0f, hi = 0.0f;
        for (int i = 0; i < 32; ++i) { lo = fminf(lo, x[32 * j + i]); hi = fmaxf(hi, x[32 * j + i]); }
        scale[j] = (hi - lo) / 15.0f;
        mn[j] = -lo;
        smax = fmaxf(smax, scale[j]);
        mmax = fmaxf(mmax, mn[j]);
    }
    const uint16_t hd = f2h_bits(smax / 63.0f), hm = f2h_bits(mmax / 63.0f);
    const float d = h2f_bits(hd), dmin = h2f_bits(hm);
    memset(o, 0, 144);
    memcpy(o, &hd, 2);
    memcpy(o + 2, &hm, 2);
    uint8_t* s12 = o + 4;
    uint8_t* qs = o + 16;
    for (int j = 0; j < 8; ++j) {
        const int sc = d > 0.0f ? iround_clamp(scale[j] / d, 0, 63) : 0;
        const int m = dmin > 0.0f ? iround_clamp(mn[j] / dmin, 0, 63) : 0;
        if (j < 4) { s12[j] |= (uint8_t) sc; s12[j + 4] |= (uint8_t) m; }
        else {
            s12[j + 4] |= (uint8_t) ((sc & 0x0F) | ((m & 0x0F) << 4));
            s12[j - 4] |= (uint8_t) ((sc >> 4) << 6);
            s12[j] |= (uint8_t) ((m >> 4) << 6);
        }
        const float dl = d * (float) sc, ml = dmin * (float) m;
        for (int i = 0; i < 32; ++i) {
            const int q = dl > 0.0f ? iround_clamp((x[32 * j + i] + ml) / dl, 0, 15) : 0;
            qs[32 * (j / 2) + i] |= (uint8_t) ((j & 1) ? (q << 4) : q);
        }
    }
}

void host_iq2_s(const float* x, uint8_t* o) {
    float db[16], dbmax = 0.0f;
    for (int h = 0; h < 16; ++h) {
        float amax = 0.0f;
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(x[16 * h + i]));
        db[h] = amax / 43.0f;
        dbmax = fmaxf(dbmax, db[h]);
    }
    const uint16_t hd = f2h_bits(dbmax * 4.0f / 15.5f);
    const float d = h2f_bits(hd);
    memset(o, 0, 82);
    memcpy(o, &hd, 2);
    uint8_t *qs = o + 2, *sg = o + 34, *qh = o + 66, *sc = o + 74;
    for (int h = 0; h < 16; ++h) {
        const int ls = d > 0.0f ? iround_clamp(4.0f * db[h] / d - 0.5f, 0, 15) : 0;
        sc[h / 2] |= (uint8_t) ((h & 1) ? (ls << 4) : ls);
        const float dl = d * (0.5f + (float) ls) * 0.25f, idl = dl > 0.0f ? 1.0f / dl : 0.0f;
        for (int g = 0; g < 2; ++g) {
            const int l = 2 * h + g;   // group of 8 weights
            float a[8];
            uint8_t s = 0;
            for (int i = 0; i < 8; ++i) {
                const float v = x[8 * l + i];
                a[i] = fabsf(v) * idl;
                if (v < 0.0f) s |= (uint8_t) (1u << i);
            }
            const int idx = nearest_iq2s(a);
            qs[l] = (uint8_t) (idx & 0xFF);
            qh[l / 4] |= (uint8_t) ((idx >> 8) << (2 * (l % 4)));
            sg[l] = s;
        }
    }
}

void host_iq3_s(const float* x, uint8_t* o) {
    float db[8], dbmax = 0.0f;
    for (int b = 0; b < 8; ++b) {
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(x[32 * b + i]));
        db[b] = amax / 15.0f;
        dbmax = fmaxf(dbmax, db[b]);
    }
    const uint16_t hd = f2h_bits(dbmax / 31.0f);
    const float d = h2f_bits(hd);
    memset(o, 0, 110);
    memcpy(o, &hd, 2);
    uint8_t *qs = o + 2, *qh = o + 66, *sg = o + 74, *sc = o + 106;
    for (int b = 0; b < 8; ++b) {
        const int ls = d > 0.0f ? iround_clamp((db[b] / d - 1.0f) * 0.5f, 0, 15) : 0;
        sc[b / 2] |= (uint8_t) ((b & 1) ? (ls << 4) : ls);
        const float dl = d * (float) (1 + 2 * ls), idl = dl > 0.0f ? 1.0f / dl : 0.0f;
        for (int l = 0; l < 8; ++l) {   // codeword of 4 weights
            float a[4];
            for (int i = 0; i < 4; ++i) {
                const float v = x[32 * b + 4 * l + i];
                a[i] = fabsf(v) * idl;
                if (v < 0.0f) sg[4 * b + l / 2] |= (uint8_t) (1u << (4 * (l & 1) + i));
            }
            const int idx = nearest_iq3s(a);
            qs[8 * b + l] = (uint8_t) (idx & 0xFF);
            qh[b] |= (uint8_t) ((idx >> 8) << l);
        }
    }
}

// ---------------------------------------------------------------- device: one warp per 256 values
template<int W> __device__ __forceinline__ float group_max(float v) {   // max over aligned groups of W lanes
#pragma unroll
    for (int o = W / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
template<int W> __device__ __forceinline__ float group_min(float v) {
#pragma unroll
    for (int o = W / 2; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
template<int W> __device__ __forceinline__ uint32_t group_or(uint32_t v) {
#pragma unroll
    for (int o = W / 2; o > 0; o >>= 1) v |= __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template<int T>
__global__ void __launch_bounds__(256) synth_kernel(uint64_t seed, float sigma, int64_t n_super, uint8_t* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t sb = (int64_t) blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (sb >= n_super) return;
    float x[8];
    float amax8 = 0.0f, lo8 = 0.0f, hi8 = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        x[i] = sigma * normal_at(seed, (uint64_t) sb * 256 + 8 * lane + i);
        amax8 = fmaxf(amax8, fabsf(x[i]));
        lo8 = fminf(lo8, x[i]);
        hi8 = fmaxf(hi8, x[i]);
    }
    if constexpr (T == MAYA_Q8_0) {
        uint8_t* o = out + (size_t) sb * 8 * 34 + (size_t) (lane >> 2) * 34;
        const uint16_t hd = f2h_bits(group_max<4>(amax8) / 127.0f);
        const float d = h2f_bits(hd), id = d > 0.0f ? 1.0f / d : 0.0f;
        if ((lane & 3) == 0) *(uint16_t*) o = hd;
#pragma unroll
        for (int i = 0; i < 8; ++i) o[2 + 8 * (lane & 3) + i] = (uint8_t) (int8_t) iround_clamp(x[i] * id, -127, 127);
    } else if constexpr (T == MAYA_Q4_K) {
        uint8_t* o = out + (size_t) sb * 144;
        const int j = lane >> 2;
        const float lo = group_min<4>(lo8), hi = group_max<4>(hi8);
        const float scale = (hi - lo) / 15.0f, mn = -lo;
        const uint16_t hd = f2h_bits(group_max<32>(scale) / 63.0f), hm = f2h_bits(group_max<32>(mn) / 63.0f);
        const float d = h2f_bits(hd), dmin = h2f_bits(hm);
        const int sc = d > 0.0f ? iround_clamp(scale / d, 0, 63) : 0;
        const int m = dmin > 0.0f ? iround_clamp(mn / dmin, 0, 63) : 0;
        // scales: gather the 8 (sc, m) pairs on lane 0 and pack the 12 bytes
        uint32_t scs[8], ms[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) { scs[q] = __shfl_sync(0xffffffffu, sc, 4 * q); ms[q] = __shfl_sync(0xffffffffu, m, 4 * q); }
        if (lane == 0) {
            *(uint16_t*) o = hd;
            *(uint16_t*) (o + 2) = hm;
            uint8_t* s12 = o + 4;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                s12[q] = (uint8_t) (scs[q] | ((scs[q + 4] >> 4) << 6));
                s12[q + 4] = (uint8_t) (ms[q] | ((ms[q + 4] >> 4) << 6));
                s12[q + 8] = (uint8_t) ((scs[q + 4] & 0x0F) | ((ms[q + 4] & 0x0F) << 4));
            }
        }
        const float dl = d * (float) sc, ml = dmin * (float) m;
        uint32_t nib[2] = {0u, 0u};   // 8 nibbles as two words of 4 bytes (low nibble of each byte)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t q = dl > 0.0f ? (uint32_t) iround_clamp((x[i] + ml) / dl, 0, 15) : 0u;
            nib[i >> 2] |= q << (8 * (i & 3));
        }
        // sub-block j even holds the low nibbles, j + 1 (lane + 4) the high nibbles of the same bytes
        const uint32_t p0 = __shfl_down_sync(0xffffffffu, nib[0], 4), p1 = __shfl_down_sync(0xffffffffu, nib[1], 4);
        if ((j & 1) == 0) {
            uint32_t* dst = (uint32_t*) (o + 16 + 32 * (j >> 1) + 8 * (lane & 3));
            dst[0] = nib[0] | (p0 << 4);
            dst[1] = nib[1] | (p1 << 4);
        }
    } else if constexpr (T == MAYA_IQ2_S) {
        uint8_t* o = out + (size_t) sb * 82;
        const float db = group_max<2>(amax8) / 43.0f;   // per 16 values
        const uint16_t hd = f2h_bits(group_max<32>(db) * 4.0f / 15.5f);
        const float d = h2f_bits(hd);
        const int ls = d > 0.0f ? iround_clamp(4.0f * db / d - 0.5f, 0, 15) : 0;
        const float dl = d * (0.5f + (float) ls) * 0.25f, idl = dl > 0.0f ? 1.0f / dl : 0.0f;
        float a[8];
        uint32_t s = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) { a[i] = fabsf(x[i]) * idl; if (x[i] < 0.0f) s |= 1u << i; }
        const int idx = nearest_iq2s(a);
        o[2 + lane] = (uint8_t) (idx & 0xFF);
        o[34 + lane] = (uint8_t) s;
        const uint32_t qh = group_or<4>((uint32_t) (idx >> 8) << (2 * (lane & 3)));
        // scale byte of sub-block lane/4: low nibble = lanes 4b, 4b+1 (first 16 values), high = lanes 4b+2, 4b+3
        const uint32_t scb = group_or<4>((uint32_t) ls << (4 * ((lane >> 1) & 1)));
        if ((lane & 3) == 0) { o[66 + (lane >> 2)] = (uint8_t) qh; o[74 + (lane >> 2)] = (uint8_t) scb; }
        if (lane == 0) *(uint16_t*) o = hd;
    } else {
        uint8_t* o = out + (size_t) sb * 110;
        const float db = group_max<4>(amax8) / 15.0f;   // per 32 values
        const uint16_t hd = f2h_bits(group_max<32>(db) / 31.0f);
        const float d = h2f_bits(hd);
        const int ls = d > 0.0f ? iround_clamp((db / d - 1.0f) * 0.5f, 0, 15) : 0;
        const float dl = d * (float) (1 + 2 * ls), idl = dl > 0.0f ? 1.0f / dl : 0.0f;
        float a[8];
        uint32_t s = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) { a[i] = fabsf(x[i]) * idl; if (x[i] < 0.0f) s |= 1u << i; }
        const int i0 = nearest_iq3s(a), i1 = nearest_iq3s(a + 4);
        o[2 + 2 * lane] = (uint8_t) (i0 & 0xFF);
        o[2 + 2 * lane + 1] = (uint8_t) (i1 & 0xFF);
        o[74 + lane] = (uint8_t) s;
        const uint32_t qh = group_or<4>((uint32_t) ((i0 >> 8) | ((i1 >> 8) << 1)) << (2 * (lane & 3)));
        if ((lane & 3) == 0) o[66 + (lane >> 2)] = (uint8_t) qh;
        // scales[b / 2]: low nibble sub-block b even, high nibble b odd; b = lane / 4
        const uint32_t scb = group_or<8>((lane & 3) == 0 ? ((uint32_t) ls << (4 * ((lane >> 2) & 1))) : 0u);
        if ((lane & 7) == 0) o[106 + (lane >> 3)] = (uint8_t) scb;
        if (lane == 0) *(uint16_t*) o = hd;
    }
}

}  // namespace
}  // namespace maya

using namespace maya;

extern "C" int maya_quantize_weights_host(int type, const float* w, int64_t n_rows, int64_t n_cols, void* out) {
    const int qk = type_qk(type);
    if (!type_is_core(type)) return MAYA_ERR_TYPE;      // quantizers exist for Q8_0, Q4_K, IQ2_S, IQ3_S only
    if (!w || !out || n_rows <= 0 || n_cols <= 0 || n_cols % qk) return MAYA_ERR_ARG;
    const int64_t nb = n_rows * (n_cols / qk);
    const int bb = type_bytes(type);
    uint8_t* o = (uint8_t*) out;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b) {
        switch (type) {
            case MAYA_Q8_0: host_q8_0(w + b * 32, o + b * bb); break;
            case MAYA_Q4_K: host_q4_K(w + b * 256, o + b * bb); break;
            case MAYA_IQ2_S: host_iq2_s(w + b * 256, o + b * bb); break;
            default: host_iq3_s(w + b * 256, o + b * bb); break;
        }
    }
    return MAYA_OK;
}

extern "C" int maya_synth_weights(int type, uint64_t seed, float sigma, int64_t n_rows, int64_t n_cols, void* out,
                                  void* stream) {
    if (!type_is_core(type)) return refuse(MAYA_ERR_TYPE);
    if (!out || n_rows <= 0 || n_cols <= 0 || n_cols % 256) return refuse(MAYA_ERR_ARG);
    const int64_t n_super = n_rows * (n_cols / 256);
    if (n_super > (int64_t) 0x7fffffff * 8) return refuse(MAYA_ERR_LIMIT);
    const unsigned grid = (unsigned) ((n_super + 7) / 8);
    cudaStream_t s = as_stream(stream);
    switch (type) {
        case MAYA_Q8_0: synth_kernel<MAYA_Q8_0><<<grid, 256, 0, s>>>(seed, sigma, n_super, (uint8_t*) out); break;
        case MAYA_Q4_K: synth_kernel<MAYA_Q4_K><<<grid, 256, 0, s>>>(seed, sigma, n_super, (uint8_t*) out); break;
        case MAYA_IQ2_S: synth_kernel<MAYA_IQ2_S><<<grid, 256, 0, s>>>(seed, sigma, n_super, (uint8_t*) out); break;
        default: synth_kernel<MAYA_IQ3_S><<<grid, 256, 0, s>>>(seed, sigma, n_super, (uint8_t*) out); break;
    }
    return note_launch("synth_weights");
}
