/*
 * maya_oracle.c - CPU restatement of the reference's routed-MoE expert-FFN arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared with.  Nothing in the
 * shipped library links, loads or calls it; only the test-suite, the smoke check and the benchmark's CPU
 * baseline leg do.  It is scalar C on purpose: every function states, next to its name, the reference
 * file:line whose arithmetic (integer grouping, rounding points, summation order) it follows.
 *
 * Parity pins (see tests/test_oracle_pins.py): the dequantizers against gguf-py's numpy dequantizers on
 * random valid blocks; the router against the host reference of the reference's own router test, built from
 * the reference sources; the quantized row dots against the reference's AVX-512/AVX2 CPU rows (IQ2_S, IQ3_S,
 * Q4_K) within float tolerance; the whole expert against a double-precision dequantize-and-dot.
 *
 * GGUF block layouts (little-endian, packed, from the GGUF format definition):
 *   Q8_0  34 B / 32 : f16 d | i8 q[32]
 *   Q8_1  36 B / 32 : f16 d | f16 s | i8 q[32]                   (activations)
 *   Q4_K 144 B / 256: f16 d | f16 dmin | u8 scales[12] | u8 qs[128]
 *   IQ2_S 82 B / 256: f16 d | u8 qs[32] | u8 signs[32] | u8 qh[8] | u8 scales[8]
 *   IQ3_S 110 B / 256: f16 d | u8 qs[64] | u8 qh[8] | u8 signs[32] | u8 scales[4]
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define MAYA_GRID_QUAL static const
#define MAYA_IQ2XXS_GRID MAYA_IQ2XXS_GRID
#define MAYA_IQ3XXS_GRID MAYA_IQ3XXS_GRID
#define MAYA_IQ1S_GRID MAYA_IQ1S_GRID
#include "maya_iq_grids.inc"

#define ORC_API __attribute__((visibility("default")))

enum { T_Q8_0 = 8, T_Q4_K = 12, T_IQ3_S = 21, T_IQ2_S = 22, T_Q5_K = 13, T_Q6_K = 14, T_IQ2_XXS = 16, T_IQ3_XXS = 18, T_IQ1_S = 19, T_IQ4_XS = 23 };

/* ------------------------------------------------------------------ small helpers */
static inline float h2f(uint16_t h) { _Float16 v; memcpy(&v, &h, 2); return (float) v; }
static inline uint16_t f2h(float f) { _Float16 v = (_Float16) f; uint16_t h; memcpy(&h, &v, 2); return h; }
static inline uint16_t rd16(const uint8_t* p) { uint16_t v; memcpy(&v, p, 2); return v; }
static inline int32_t rd32(const uint8_t* p) { int32_t v; memcpy(&v, p, 4); return v; }

/* 4 signed bytes x 4 signed bytes + c: CUDA's __dp4a(int, int, int). */
static inline int dp4a(int a, int b, int c) {
    for (int i = 0; i < 4; ++i) c += (int) (int8_t) (a >> (8 * i)) * (int) (int8_t) (b >> (8 * i));
    return c;
}

/* butterfly sum over 32 lanes: x += shfl_xor(x, 16), 8, 4, 2, 1 (native_mmvq.cu:124-130, glm_fast.cu:66-70).
 * Every lane ends with the same bits because float addition commutes; lane 0's value is returned. */
static float warp_tree_sum(const float* lane) {
    float v[32];
    memcpy(v, lane, sizeof v);
    for (int off = 16; off > 0; off >>= 1) {
        float n[32];
        for (int l = 0; l < 32; ++l) n[l] = v[l] + v[l ^ off];
        memcpy(v, n, sizeof v);
    }
    return v[0];
}

ORC_API int orc_type_block_bytes(int type) {
    switch (type) {
        case T_Q8_0: return 34; case T_Q4_K: return 144; case T_IQ3_S: return 110; case T_IQ2_S: return 82;
        case T_Q5_K: return 176; case T_Q6_K: return 210; case T_IQ4_XS: return 136; case T_IQ3_XXS: return 98; case T_IQ2_XXS: return 66; case T_IQ1_S: return 50;
        default: return 0;
    }
}
ORC_API int orc_type_block_values(int type) { return type == T_Q8_0 ? 32 : orc_type_block_bytes(type) ? 256 : 0; }
/* iq_row_bytes (iq_kernels.cu:984-1006) / native_mmvq_weight_bytes (native_mmvq.cu). */
ORC_API size_t orc_row_bytes(int type, int64_t n) {
    const int bv = orc_type_block_values(type);
    return bv ? (size_t) (n / bv) * (size_t) orc_type_block_bytes(type) : 0;
}

/* ------------------------------------------------------------------ q8_1 activations
 * native_quantize_q8_1_kernel (native_mmvq.cu:140-152) == q8_1_store_warp (glm_fast.cu:165-174):
 * per 32 values amax by max, sum by the butterfly tree over the ORIGINAL floats, d = min(amax/127, 65504),
 * q = round-half-away(x / d) clamped to +-127, stored {f16 d, f16 clamp(sum)}.  The reference divides with
 * the GPU's fast-math reciprocal in one of its two translation units; this uses IEEE division. */
ORC_API void orc_quantize_q8_1(const float* x, uint8_t* y, int64_t n) {
    for (int64_t b = 0; b < n / 32; ++b) {
        const float* xb = x + 32 * b;
        uint8_t* o = y + 36 * b;
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(xb[i]));
        const float sum = warp_tree_sum(xb);
        const float d = fminf(amax / 127.0f, 65504.0f);
        for (int i = 0; i < 32; ++i) {
            const float q = amax == 0.0f ? 0.0f : fmaxf(-127.0f, fminf(127.0f, roundf(xb[i] / d)));
            o[4 + i] = (uint8_t) (int8_t) q;
        }
        const uint16_t hd = f2h(d), hs = f2h(fmaxf(-65504.0f, fminf(65504.0f, sum)));
        memcpy(o, &hd, 2);
        memcpy(o + 2, &hs, 2);
    }
}

/* ------------------------------------------------------------------ dequantizers (double-checked against gguf-py) */
static void q4k_scale_min(const uint8_t* sc12, int j, int* sc, int* mn) {
    if (j < 4) { *sc = sc12[j] & 63; *mn = sc12[j + 4] & 63; }
    else { *sc = (sc12[j + 4] & 0x0F) | ((sc12[j - 4] >> 6) << 4); *mn = (sc12[j + 4] >> 4) | ((sc12[j] >> 6) << 4); }
}

static void dequant_block(int type, const uint8_t* b, float* y) {
    if (type == T_Q8_0) {
        const float d = h2f(rd16(b));
        for (int i = 0; i < 32; ++i) y[i] = d * (float) (int8_t) b[2 + i];
    } else if (type == T_Q4_K) {
        const float d = h2f(rd16(b)), dmin = h2f(rd16(b + 2));
        const uint8_t* qs = b + 16;
        for (int j = 0; j < 8; ++j) {
            int sc, mn;
            q4k_scale_min(b + 4, j, &sc, &mn);
            const float dl = d * (float) sc, ml = dmin * (float) mn;
            for (int i = 0; i < 32; ++i) {
                const int q = (j & 1) ? (qs[32 * (j / 2) + i] >> 4) : (qs[32 * (j / 2) + i] & 0x0F);
                y[32 * j + i] = dl * (float) q - ml;
            }
        }
    } else if (type == T_IQ2_S) {
        const float d = h2f(rd16(b));
        const uint8_t *qs = b + 2, *sg = b + 34, *qh = b + 66, *sc = b + 74;
        for (int ib = 0; ib < 8; ++ib) {
            for (int l = 0; l < 4; ++l) {
                const int ls = l < 2 ? (sc[ib] & 0x0F) : (sc[ib] >> 4);
                const float db = d * (0.5f + (float) ls) * 0.25f;
                const int idx = qs[4 * ib + l] | (((qh[ib] >> (2 * l)) & 3) << 8);
                const uint64_t g = MAYA_IQ2S_GRID[idx];
                const uint8_t s = sg[4 * ib + l];
                for (int j = 0; j < 8; ++j) {
                    const float v = db * (float) ((g >> (8 * j)) & 0xFF);
                    y[32 * ib + 8 * l + j] = ((s >> j) & 1) ? -v : v;
                }
            }
        }
    } else if (type == T_IQ3_S) {
        const float d = h2f(rd16(b));
        const uint8_t *qs = b + 2, *qh = b + 66, *sg = b + 74, *sc = b + 106;
        for (int ib = 0; ib < 8; ++ib) {
            const int ls = (sc[ib / 2] >> (4 * (ib & 1))) & 0x0F;
            const float db = d * (float) (1 + 2 * ls);
            for (int l = 0; l < 8; ++l) {
                const int idx = qs[8 * ib + l] | (((qh[ib] >> l) & 1) << 8);
                const uint32_t g = MAYA_IQ3S_GRID[idx];
                const uint8_t s = sg[4 * ib + l / 2];
                for (int j = 0; j < 4; ++j) {
                    const float v = db * (float) ((g >> (8 * j)) & 0xFF);
                    y[32 * ib + 4 * l + j] = ((s >> (4 * (l & 1) + j)) & 1) ? -v : v;
                }
            }
        }
    } else if (type == T_Q5_K) {
        /* dequantize_row_q5_K (ggml-quants.c): Q4_K's layout with qh[32] between the scales and qs; bit sb of qh[l] is
         * the fifth bit of value l of sub-block sb. */
        const float d = h2f(rd16(b)), dmin = h2f(rd16(b + 2));
        const uint8_t *qh = b + 16, *qs = b + 48;
        for (int j = 0; j < 8; ++j) {
            int sc, mn;
            q4k_scale_min(b + 4, j, &sc, &mn);
            const float dl = d * (float) sc, ml = dmin * (float) mn;
            for (int i = 0; i < 32; ++i) {
                const int q4 = (j & 1) ? (qs[32 * (j / 2) + i] >> 4) : (qs[32 * (j / 2) + i] & 0x0F);
                const int q = q4 | (((qh[i] >> j) & 1) << 4);
                y[32 * j + i] = dl * (float) q - ml;
            }
        }
    } else if (type == T_Q6_K) {
        /* dequantize_row_q6_K: ql[128] | qh[64] | int8 scales[16] | f16 d; run r = 4 h + k of 32 values. */
        const float d = h2f(rd16(b + 208));
        const int8_t* sc = (const int8_t*) (b + 192);
        for (int r = 0; r < 8; ++r) {
            const int h = r >> 2, k = r & 3;
            const uint8_t *ql = b + 64 * h + 32 * (k & 1), *qh = b + 128 + 32 * h;
            for (int l = 0; l < 32; ++l) {
                const int q = (((k >> 1) ? (ql[l] >> 4) : (ql[l] & 0x0F)) | (((qh[l] >> (2 * k)) & 3) << 4)) - 32;
                y[32 * r + l] = (d * (float) sc[8 * h + 2 * k + l / 16]) * (float) q;
            }
        }
    } else if (type == T_IQ4_XS) {
        /* dequantize_row_iq4_xs: f16 d | u16 scales_h | u8 scales_l[4] | qs[128]; y = d (ls - 32) kvalues[q]. */
        static const int8_t kv[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
        const float d = h2f(rd16(b));
        const int sh = rd16(b + 2);
        for (int ib = 0; ib < 8; ++ib) {
            const int ls = ((b[4 + ib / 2] >> (4 * (ib & 1))) & 0x0F) | (((sh >> (2 * ib)) & 3) << 4);
            const float dl = d * (float) (ls - 32);
            const uint8_t* qs = b + 8 + 16 * ib;
            for (int j = 0; j < 16; ++j) {
                y[32 * ib + j] = dl * (float) kv[qs[j] & 0x0F];
                y[32 * ib + 16 + j] = dl * (float) kv[qs[j] >> 4];
            }
        }
    } else if (type == T_IQ3_XXS) {
        /* dequantize_row_iq3_xxs: f16 d | qs[64] | u32 gas[8]: db = d (0.5 + (gas >> 28)) 0.5; 7 sign bits per 8 values, the
         * eighth from their parity (ksigns_iq2xs). */
        const float d = h2f(rd16(b));
        for (int ib = 0; ib < 8; ++ib) {
            const uint32_t aux = (uint32_t) rd32(b + 66 + 4 * ib);
            const float db = d * (0.5f + (float) (aux >> 28)) * 0.5f;
            for (int l = 0; l < 4; ++l) {
                const uint32_t s7 = (aux >> (7 * l)) & 127u;
                const uint32_t s8 = s7 | ((uint32_t) (__builtin_popcount(s7) & 1) << 7);
                for (int e = 0; e < 2; ++e) {
                    const uint32_t g = MAYA_IQ3XXS_GRID[b[2 + 8 * ib + 2 * l + e]];
                    for (int j = 0; j < 4; ++j) {
                        const float v = db * (float) ((g >> (8 * j)) & 0xFF);
                        y[32 * ib + 8 * l + 4 * e + j] = ((s8 >> (4 * e + j)) & 1) ? -v : v;
                    }
                }
            }
        }
    } else if (type == T_IQ2_XXS) {
        /* dequantize_row_iq2_xxs: f16 d | per 32 values { u8 idx[4] | u32 aux }: db = d (0.5 + (aux >> 28)) 0.25. */
        const float d = h2f(rd16(b));
        for (int ib = 0; ib < 8; ++ib) {
            const uint8_t* q = b + 2 + 8 * ib;
            const uint32_t aux = (uint32_t) rd32(q + 4);
            const float db = d * (0.5f + (float) (aux >> 28)) * 0.25f;
            for (int l = 0; l < 4; ++l) {
                const uint32_t s7 = (aux >> (7 * l)) & 127u;
                const uint32_t s8 = s7 | ((uint32_t) (__builtin_popcount(s7) & 1) << 7);
                const uint64_t g = MAYA_IQ2XXS_GRID[q[l]];
                for (int j = 0; j < 8; ++j) {
                    const float v = db * (float) ((g >> (8 * j)) & 0xFF);
                    y[32 * ib + 8 * l + j] = ((s8 >> j) & 1) ? -v : v;
                }
            }
        }
    } else if (type == T_IQ1_S) {
        /* dequantize_row_iq1_s: f16 d | qs[32] | u16 qh[8]: dl = d (2 ((qh >> 12) & 7) + 1), delta = +-0.125 by qh bit 15,
         * index = qs | ((qh >> 3l) & 7) << 8, y = dl (g + delta) with g in {-1, 0, 1} (the table holds g + 1 in nibbles:
         * byte j low = value j, high = value j + 4). */
        const float d = h2f(rd16(b));
        for (int ib = 0; ib < 8; ++ib) {
            const int qh = rd16(b + 34 + 2 * ib);
            const float dl = d * (float) (2 * ((qh >> 12) & 7) + 1), delta = (qh & 0x8000) ? -0.125f : 0.125f;
            for (int l = 0; l < 4; ++l) {
                const uint32_t g = MAYA_IQ1S_GRID[b[2 + 4 * ib + l] | (((qh >> (3 * l)) & 7) << 8)];
                for (int j = 0; j < 8; ++j) {
                    const int v = (int) ((g >> (8 * (j & 3) + 4 * (j >> 2))) & 0x0F) - 1;
                    y[32 * ib + 8 * l + j] = dl * ((float) v + delta);
                }
            }
        }
    }
}

ORC_API int orc_dequantize(int type, const uint8_t* w, int64_t n, float* y) {
    const int bv = orc_type_block_values(type), bb = orc_type_block_bytes(type);
    if (!bv || n % bv) return -1;
    for (int64_t i = 0; i < n / bv; ++i) dequant_block(type, w + i * bb, y + i * bv);
    return 0;
}

/* ------------------------------------------------------------------ the quantized dot, one "call" at a time
 *
 * The reference's GPU dots are organised as calls: a call covers `8 or 16` weights of one block against the
 * q8_1 block(s) they meet and returns a float.  glm_fast.cu's F<T> table (:624-645) gives calls per block:
 * Q8_0 4 (8 weights each), Q4_K 16 (16 weights), IQ2_S / IQ3_S 8 (32 weights).  xq points at the q8_1 block of
 * the weight block's FIRST value. */
static int calls_per_block(int type) { return type == T_Q8_0 ? 4 : type == T_Q4_K ? 16 : 8; }

/* vec_dot_q8_0_q8_1 (native_mmvq.cu:708-720; glm_fast.cu:336-345): call c covers ints 2c, 2c+1. */
static float call_q8_0(const uint8_t* b, const uint8_t* xq, int c) {
    int sumi = 0;
    for (int i = 0; i < 2; ++i) sumi = dp4a(rd32(b + 2 + 4 * (2 * c + i)), rd32(xq + 4 + 4 * (2 * c + i)), sumi);
    return h2f(rd16(b)) * h2f(rd16(xq)) * (float) sumi;
}

/* vec_dot_q4_K_q8_1 with llama.cpp's _impl_vmmq order (native_mmvq.cu:495-547; glm_fast.cu:206-243).
 * Call c (iqs = 2c): 64-value group j = c/4 (sub-blocks 2j: low nibbles, 2j+1: high nibbles of qs[32j..]),
 * bytes p..p+3 and p+16..p+19 with p = 4*(c%4). */
static float call_q4_K(const uint8_t* b, const uint8_t* xq, int c) {
    const int j = c / 4, p = 4 * (c % 4);
    const uint8_t* qs = b + 16 + 32 * j;
    const int v0 = rd32(qs + p), v1 = rd32(qs + p + 16);
    float sumf_d = 0.0f, sumf_m = 0.0f;
    for (int i = 0; i < 2; ++i) {
        int sc, mn;
        q4k_scale_min(b + 4, 2 * j + i, &sc, &mn);
        const uint8_t* q8 = xq + 36 * (2 * j + i);
        const float d8 = h2f(rd16(q8));
        const int u0 = rd32(q8 + 4 + p), u1 = rd32(q8 + 4 + p + 16);
        const int v0i = (v0 >> (4 * i)) & 0x0F0F0F0F, v1i = (v1 >> (4 * i)) & 0x0F0F0F0F;
        const int dot1 = dp4a(v1i, u1, dp4a(v0i, u0, 0));
        const int dot2 = dp4a(0x01010101, u1, dp4a(0x01010101, u0, 0));
        sumf_d = fmaf(d8, (float) (dot1 * sc), sumf_d);
        sumf_m = fmaf(d8, (float) (dot2 * mn), sumf_m);
    }
    const float d = h2f(rd16(b)), dmin = h2f(rd16(b + 2));
    return d * sumf_d - dmin * sumf_m;
}

/* vec_dot_iq2_s_q8_1 (iq_kernels.cu:138-169; glm_fast.cu:927-962): call c covers sub-block c (32 weights),
 * two 16-weight halves with their own 4-bit scale, combined with truncating integer division. */
static float call_iq2_s(const uint8_t* b, const uint8_t* xq, int c) {
    const uint8_t *qs = b + 2, *sg = b + 34, *qh = b + 66, *sc = b + 74;
    const uint8_t* q8 = xq + 36 * c;
    const int ls0 = sc[c] & 0x0F, ls1 = sc[c] >> 4;
    int sumi0 = 0, sumi1 = 0;
    for (int l = 0; l < 4; ++l) {
        const int idx = qs[4 * c + l] | (((qh[c] >> (2 * l)) & 3) << 8);
        const uint64_t g = MAYA_IQ2S_GRID[idx];
        const uint8_t s = sg[4 * c + l];
        int part = 0;
        for (int j = 0; j < 8; ++j) {
            const int w = (int) ((g >> (8 * j)) & 0xFF);
            part += (((s >> j) & 1) ? -w : w) * (int) (int8_t) q8[4 + 8 * l + j];
        }
        if (l < 2) sumi0 += part; else sumi1 += part;
    }
    const int sumi = (sumi0 * ls0 + sumi1 * ls1 + (sumi0 + sumi1) / 2) / 4;
    return h2f(rd16(b)) * h2f(rd16(q8)) * (float) sumi;
}

/* vec_dot_iq3_s_q8_1 (iq_kernels.cu:197-222; glm_fast.cu:963-991): call c covers sub-block c. */
static float call_iq3_s(const uint8_t* b, const uint8_t* xq, int c) {
    const uint8_t *qs = b + 2, *qh = b + 66, *sg = b + 74, *sc = b + 106;
    const uint8_t* q8 = xq + 36 * c;
    int sumi = 0;
    for (int l = 0; l < 8; ++l) {
        const int idx = qs[8 * c + l] | (((qh[c] >> l) & 1) << 8);
        const uint32_t g = MAYA_IQ3S_GRID[idx];
        const uint8_t s = sg[4 * c + l / 2];
        for (int j = 0; j < 4; ++j) {
            const int w = (int) ((g >> (8 * j)) & 0xFF);
            sumi += (((s >> (4 * (l & 1) + j)) & 1) ? -w : w) * (int) (int8_t) q8[4 + 4 * l + j];
        }
    }
    sumi *= 1 + 2 * ((sc[c / 2] >> (4 * (c & 1))) & 0x0F);
    return h2f(rd16(b)) * h2f(rd16(q8)) * (float) sumi;
}

/* The other block types of glmf::moe_supported (glm_fast.cu:5798-5801), one 32-weight sub-block a call.  The integer
 * sums are llama.cpp's vec_dot_*_q8_1 as glm_fast.cu transcribes them (dot_q5_K :246-290, dot_q6_K :310-335, dot_iq2_xxs
 * :536-559, dot_iq3_xxs :560-583, dot_iq4_xs :605-621): exact int8 dots, Q5_K's scale and min terms with the sum of the
 * activation quants, Q6_K's two int8 scales per 32 values, IQ4_XS's (ls - 32) * sum, IQ3_XXS's (ls * s + s / 2) / 2 and
 * IQ2_XXS's s * (2 ls + 1) / 8 with truncating division. */
static int signed_dot8(uint64_t g, uint32_t s8, const uint8_t* q8) {
    int part = 0;
    for (int j = 0; j < 8; ++j) {
        const int w = (int) ((g >> (8 * j)) & 0xFF);
        part += (((s8 >> j) & 1) ? -w : w) * (int) (int8_t) q8[j];
    }
    return part;
}
static float call_q5_K(const uint8_t* b, const uint8_t* xq, int sb) {
    const uint8_t *qh = b + 16, *qs = b + 48 + 32 * (sb / 2), *q8 = xq + 36 * sb;
    int sc, mn, dot1 = 0, dot2 = 0;
    q4k_scale_min(b + 4, sb, &sc, &mn);
    for (int i = 0; i < 32; ++i) {
        const int q = ((sb & 1) ? (qs[i] >> 4) : (qs[i] & 0x0F)) | (((qh[i] >> sb) & 1) << 4);
        dot1 += q * (int) (int8_t) q8[4 + i];
        dot2 += (int) (int8_t) q8[4 + i];
    }
    const float d8 = h2f(rd16(q8));
    return h2f(rd16(b)) * (d8 * (float) (dot1 * sc)) - h2f(rd16(b + 2)) * (d8 * (float) (dot2 * mn));
}
static float call_q6_K(const uint8_t* b, const uint8_t* xq, int r) {
    const int h = r >> 2, k = r & 3;
    const uint8_t *ql = b + 64 * h + 32 * (k & 1), *qh = b + 128 + 32 * h, *q8 = xq + 36 * r;
    const int8_t* sc = (const int8_t*) (b + 192) + 8 * h + 2 * k;
    int s[2] = {0, 0};
    for (int l = 0; l < 32; ++l) {
        const int q = (((k >> 1) ? (ql[l] >> 4) : (ql[l] & 0x0F)) | (((qh[l] >> (2 * k)) & 3) << 4)) - 32;
        s[l / 16] += q * (int) (int8_t) q8[4 + l];
    }
    return h2f(rd16(b + 208)) * h2f(rd16(q8)) * (float) (s[0] * sc[0] + s[1] * sc[1]);
}
static float call_iq4_xs(const uint8_t* b, const uint8_t* xq, int ib) {
    static const int8_t kv[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
    const int sh = rd16(b + 2);
    const int ls = (((b[4 + ib / 2] >> (4 * (ib & 1))) & 0x0F) | (((sh >> (2 * ib)) & 3) << 4)) - 32;
    const uint8_t *qs = b + 8 + 16 * ib, *q8 = xq + 36 * ib;
    int sumi = 0;
    for (int j = 0; j < 16; ++j)
        sumi += kv[qs[j] & 0x0F] * (int) (int8_t) q8[4 + j] + kv[qs[j] >> 4] * (int) (int8_t) q8[4 + 16 + j];
    return h2f(rd16(b)) * h2f(rd16(q8)) * (float) (sumi * ls);
}
static float call_iq3_xxs(const uint8_t* b, const uint8_t* xq, int ib) {
    const uint32_t aux = (uint32_t) rd32(b + 66 + 4 * ib);
    const uint8_t* q8 = xq + 36 * ib;
    int sumi = 0;
    for (int l = 0; l < 4; ++l) {
        const uint32_t s7 = (aux >> (7 * l)) & 127u;
        const uint32_t s8 = s7 | ((uint32_t) (__builtin_popcount(s7) & 1) << 7);
        const uint64_t g = (uint64_t) MAYA_IQ3XXS_GRID[b[2 + 8 * ib + 2 * l]] | ((uint64_t) MAYA_IQ3XXS_GRID[b[2 + 8 * ib + 2 * l + 1]] << 32);
        sumi += signed_dot8(g, s8, q8 + 4 + 8 * l);
    }
    const int ls = (int) (aux >> 28);
    sumi = (ls * sumi + sumi / 2) / 2;
    return h2f(rd16(b)) * h2f(rd16(q8)) * (float) sumi;
}
static float call_iq2_xxs(const uint8_t* b, const uint8_t* xq, int ib) {
    const uint8_t *q = b + 2 + 8 * ib, *q8 = xq + 36 * ib;
    const uint32_t aux = (uint32_t) rd32(q + 4);
    int sumi = 0;
    for (int l = 0; l < 4; ++l) {
        const uint32_t s7 = (aux >> (7 * l)) & 127u;
        const uint32_t s8 = s7 | ((uint32_t) (__builtin_popcount(s7) & 1) << 7);
        sumi += signed_dot8(MAYA_IQ2XXS_GRID[q[l]], s8, q8 + 4 + 8 * l);
    }
    const int ls = (int) (aux >> 27) | 1;                 /* 2 * scale + 1 (dot_iq2_xxs, glm_fast.cu:555-556) */
    sumi = sumi * ls / 8;
    return h2f(rd16(b)) * h2f(rd16(q8)) * (float) sumi;
}

/* dot_iq1_s (glm_fast.cu:584-604): sum over the sub-block of (g + 1) q, then d1q (d8 sumi + S8 delta) with S8 the q8_1
 * block's stored sum of the unquantized activations and delta = -1 + 1/8 (- 1/4 when qh bit 15 is set). */
static float call_iq1_s(const uint8_t* b, const uint8_t* xq, int ib) {
    const int qh = rd16(b + 34 + 2 * ib);
    const uint8_t* q8 = xq + 36 * ib;
    int sumi = 0;
    for (int l = 0; l < 4; ++l) {
        const uint32_t g = MAYA_IQ1S_GRID[b[2 + 4 * ib + l] | (((qh >> (3 * l)) & 7) << 8)];
        for (int j = 0; j < 8; ++j)
            sumi += (int) ((g >> (8 * (j & 3) + 4 * (j >> 2))) & 0x0F) * (int) (int8_t) q8[4 + 8 * l + j];
    }
    const float d1q = h2f(rd16(b)) * (float) (2 * ((qh >> 12) & 7) + 1);
    const float delta = (qh & 0x8000) ? -1.125f : -0.875f;
    return d1q * (h2f(rd16(q8)) * (float) sumi + h2f(rd16(q8 + 2)) * delta);
}

static float call_dot(int type, const uint8_t* blk, const uint8_t* xq, int c) {
    switch (type) {
        case T_IQ1_S: return call_iq1_s(blk, xq, c);
        case T_Q5_K: return call_q5_K(blk, xq, c);
        case T_Q6_K: return call_q6_K(blk, xq, c);
        case T_IQ4_XS: return call_iq4_xs(blk, xq, c);
        case T_IQ3_XXS: return call_iq3_xxs(blk, xq, c);
        case T_IQ2_XXS: return call_iq2_xxs(blk, xq, c);
        case T_Q8_0: return call_q8_0(blk, xq, c);
        case T_Q4_K: return call_q4_K(blk, xq, c);
        case T_IQ2_S: return call_iq2_s(blk, xq, c);
        default: return call_iq3_s(blk, xq, c);
    }
}

/* One weight row against one q8_1 column with `nthreads` partial sums (32: one warp per row, glm_fast.cu
 * row_dot :647-656 / rows_dot :1323-1364, iq_kernels.cu row_dot :439-456; 128: native_mmvq's 4-warp block,
 * native_mmvq.cu:551-589).  Call c goes to thread c % nthreads in ascending c; warps are added in ascending
 * order, then the butterfly tree. */
static float row_dot(int type, const uint8_t* row, const uint8_t* xq, int n_in, int nthreads) {
    const int bv = orc_type_block_values(type), bb = orc_type_block_bytes(type), cpb = calls_per_block(type);
    float acc[128];
    for (int i = 0; i < nthreads; ++i) acc[i] = 0.0f;
    const int ncalls = (n_in / bv) * cpb;
    for (int c = 0; c < ncalls; ++c) {
        const int kb = c / cpb;
        acc[c % nthreads] += call_dot(type, row + (size_t) kb * bb, xq + (size_t) kb * (bv / 32) * 36, c % cpb);
    }
    float lane[32];
    for (int l = 0; l < 32; ++l) {
        lane[l] = acc[l];
        for (int w = 1; w < nthreads / 32; ++w) lane[l] += acc[32 * w + l];
    }
    return warp_tree_sum(lane);
}

/* native_mmvq / iq_mmvq (native_mmvq.hpp:109, iq_kernels.hpp:24): y[c*n_out + r] = W_r . x_c.
 * order: 0 = one warp per row (iq_mmvq, glm_fast), 1 = native_mmvq's 128-thread block. */
ORC_API int orc_mmvq(int type, const uint8_t* w, const uint8_t* xq, float* y, int n_in, int n_out, int ncols, int order) {
    const int bv = orc_type_block_values(type);
    if (!bv || n_in <= 0 || n_in % bv || n_out <= 0 || ncols <= 0) return -1;
    const size_t rb = orc_row_bytes(type, n_in), cb = (size_t) (n_in / 32) * 36;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t) ncols * n_out; ++i) {
        const int c = (int) (i / n_out), r = (int) (i % n_out);
        y[i] = row_dot(type, w + (size_t) r * rb, xq + (size_t) c * cb, n_in, order ? 128 : 32);
    }
    return 0;
}

/* ------------------------------------------------------------------ SwiGLU
 * clamped (glm_fast.cu:4908-4913): g = min(g, L), u = clamp(u, -L, L), h = (g / (1 + expf(-g))) * u.
 * L = +inf gives the plain silu(g) * u of the native grouped path (iq_kernels.cu:606-613). */
static float swiglu(float g, float u, float limit) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return (g / (1.0f + expf(-g))) * u;
}
ORC_API void orc_swiglu(const float* g, const float* u, float limit, int64_t n, float* h) {
    for (int64_t i = 0; i < n; ++i) h[i] = swiglu(g[i], u[i], limit);
}

/* ------------------------------------------------------------------ one expert through the quantized path
 * moe_gate_up_kernel + moe_down_kernel for one plan entry (glm_fast.cu:4808-4915, :4923-5006):
 * gate/up rows over xq -> clamped SwiGLU -> q8_1(h) -> down rows over hq.  blob = [gate | up | down].
 * part: n_embd floats (unweighted); hq_out (optional): n_ff/32 q8_1 blocks. */
ORC_API int orc_expert_q8_1(int gu_type, int d_type, const uint8_t* blob, int n_embd, int n_ff, float limit,
                            const uint8_t* xq, float* part, uint8_t* hq_out) {
    if (!orc_type_block_values(gu_type) || !orc_type_block_values(d_type)) return -1;
    if (n_embd % orc_type_block_values(gu_type) || n_ff % orc_type_block_values(d_type) || n_ff % 32) return -1;
    const size_t grb = orc_row_bytes(gu_type, n_embd), drb = orc_row_bytes(d_type, n_ff);
    const uint8_t* up = blob + (size_t) n_ff * grb;
    const uint8_t* down = up + (size_t) n_ff * grb;
    float* h = (float*) malloc(sizeof(float) * (size_t) n_ff);
    uint8_t* hq = (uint8_t*) malloc((size_t) (n_ff / 32) * 36);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < n_ff; ++r) {
        const float g = row_dot(gu_type, blob + (size_t) r * grb, xq, n_embd, 32);
        const float u = row_dot(gu_type, up + (size_t) r * grb, xq, n_embd, 32);
        h[r] = swiglu(g, u, limit);
    }
    orc_quantize_q8_1(h, hq, n_ff);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < n_embd; ++r) part[r] = row_dot(d_type, down + (size_t) r * drb, hq, n_ff, 32);
    if (hq_out) memcpy(hq_out, hq, (size_t) (n_ff / 32) * 36);
    free(h);
    free(hq);
    return 0;
}

/* The float oracle of the reference's own expert test (native_expert_parity.cpp:69-96): weights
 * dequantized to float, products and sums in double, h rounded to float, plain (unclamped) SwiGLU. */
ORC_API int orc_expert_f64(int gu_type, int d_type, const uint8_t* blob, int n_embd, int n_ff, const float* x, float* out) {
    if (!orc_type_block_values(gu_type) || !orc_type_block_values(d_type)) return -1;
    const size_t grb = orc_row_bytes(gu_type, n_embd), drb = orc_row_bytes(d_type, n_ff);
    const uint8_t* up = blob + (size_t) n_ff * grb;
    const uint8_t* down = up + (size_t) n_ff * grb;
    float* h = (float*) malloc(sizeof(float) * (size_t) n_ff);
#pragma omp parallel
    {
        float* wrow = (float*) malloc(sizeof(float) * (size_t) (n_embd > n_ff ? n_embd : n_ff));
#pragma omp for schedule(static)
        for (int r = 0; r < n_ff; ++r) {
            double g = 0, u = 0;
            orc_dequantize(gu_type, blob + (size_t) r * grb, n_embd, wrow);
            for (int i = 0; i < n_embd; ++i) g += (double) wrow[i] * x[i];
            orc_dequantize(gu_type, up + (size_t) r * grb, n_embd, wrow);
            for (int i = 0; i < n_embd; ++i) u += (double) wrow[i] * x[i];
            h[r] = (float) (g / (1.0 + exp(-g)) * u);
        }
#pragma omp for schedule(static)
        for (int r = 0; r < n_embd; ++r) {
            double o = 0;
            orc_dequantize(d_type, down + (size_t) r * drb, n_ff, wrow);
            for (int i = 0; i < n_ff; ++i) o += (double) wrow[i] * h[i];
            out[r] = (float) o;
        }
        free(wrow);
    }
    free(h);
    return 0;
}

/* ------------------------------------------------------------------ combine
 * moe_down_kernel's tail (glm_fast.cu:4999-5005): m = 0; m += w_i * part_i (fused multiply-add, plan order);
 * out = m + shared.  parts [k][n], entries with skip[i] != 0 contribute 0 (a plan pointer of 0). */
ORC_API void orc_combine_down(const float* parts, const float* w, const uint8_t* skip, int k, const float* shared,
                              int64_t n, float* out) {
    for (int64_t r = 0; r < n; ++r) {
        float m = 0.0f;
        for (int i = 0; i < k; ++i) m = fmaf(w[i], (skip && skip[i]) ? 0.0f : parts[(size_t) i * n + r], m);
        out[r] = m + (shared ? shared[r] : 0.0f);
    }
}
/* native_moe combine (native_moe.cu:34-48): first product rounded, then an FMA chain in expert order, the
 * shared row added once afterwards. */
ORC_API void orc_combine_native(const float* parts, const float* w, int k, const float* shared, int64_t n, float* out) {
    for (int64_t r = 0; r < n; ++r) {
        float s = parts[r] * w[0];
        for (int i = 1; i < k; ++i) s = fmaf(parts[(size_t) i * n + r], w[i], s);
        out[r] = shared ? s + shared[r] : s;
    }
}

/* ------------------------------------------------------------------ routers
 * router_top10_kernel, value for value (router_top10.cu:69-187): float max; exp in double of
 * (double) l - (double) max; one ascending double sum; inv = (float) (1 / sum); p = (float) (ex * inv);
 * k rounds of arg-max with strict > scanning ascending (lowest index wins ties); weights renormalised in
 * double by max(sum, 2^-14). */
ORC_API int orc_router_top10(const float* logits, int n_tokens, int n_expert, int k, int32_t* ids, float* weights) {
    if (n_tokens <= 0 || n_expert <= 0 || k <= 0) return 0;
    if (k > 64 || k > n_expert) return -1;
    double* ex = (double*) malloc(sizeof(double) * (size_t) n_expert);
    float* p = (float*) malloc(sizeof(float) * (size_t) n_expert);
    uint8_t* taken = (uint8_t*) malloc((size_t) n_expert);
    for (int t = 0; t < n_tokens; ++t) {
        const float* l = logits + (size_t) t * n_expert;
        float mx = -INFINITY;
        for (int e = 0; e < n_expert; ++e) mx = fmaxf(mx, l[e]);
        double sum = 0.0;
        for (int e = 0; e < n_expert; ++e) { ex[e] = exp((double) l[e] - (double) mx); sum += ex[e]; }
        const float inv = (float) (1.0 / sum);
        for (int e = 0; e < n_expert; ++e) { p[e] = (float) (ex[e] * inv); taken[e] = 0; }
        for (int i = 0; i < k; ++i) {
            float bv = -INFINITY;
            int bi = n_expert;
            for (int e = 0; e < n_expert; ++e)
                if (!taken[e] && p[e] > bv) { bv = p[e]; bi = e; }
            if (bi < n_expert) { ids[(size_t) t * k + i] = bi; weights[(size_t) t * k + i] = bv; taken[bi] = 1; }
        }
        double s = 0.0;
        for (int i = 0; i < k; ++i) s += (double) weights[(size_t) t * k + i];
        const double sc = fmax(s, 6.103515625e-05);
        for (int i = 0; i < k; ++i) weights[(size_t) t * k + i] = (float) ((double) weights[(size_t) t * k + i] / sc);
    }
    free(ex); free(p); free(taken);
    return 0;
}

/* The double-precision host reference the reference's router test checks its kernel against
 * (router_top10_parity.cpp:36-60): p in double, stable descending order, weights (float) p / max(sum, 2^-14). */
ORC_API int orc_router_f64(const float* logits, int n_tokens, int n_expert, int k, int32_t* ids, float* weights) {
    double* p = (double*) malloc(sizeof(double) * (size_t) n_expert);
    uint8_t* taken = (uint8_t*) malloc((size_t) n_expert);
    for (int t = 0; t < n_tokens; ++t) {
        const float* l = logits + (size_t) t * n_expert;
        double mx = l[0];
        for (int e = 1; e < n_expert; ++e) mx = mx > (double) l[e] ? mx : (double) l[e];
        double sum = 0;
        for (int e = 0; e < n_expert; ++e) { p[e] = exp((double) l[e] - mx); sum += p[e]; }
        for (int e = 0; e < n_expert; ++e) { p[e] /= sum; taken[e] = 0; }
        double s = 0;
        for (int i = 0; i < k; ++i) {
            int bi = -1;
            for (int e = 0; e < n_expert; ++e)
                if (!taken[e] && (bi < 0 || p[e] > p[bi])) bi = e;
            taken[bi] = 1;
            ids[(size_t) t * k + i] = bi;
            weights[(size_t) t * k + i] = (float) p[bi];
            s += p[bi];
        }
        s = s > 6.103515625e-05 ? s : 6.103515625e-05;
        for (int i = 0; i < k; ++i) weights[(size_t) t * k + i] = (float) ((double) weights[(size_t) t * k + i] / s);
    }
    free(p); free(taken);
    return 0;
}

/* router_sigmoid_kernel (router_sigmoid.cu:29-74) / glmb::route_kernel (glm_batch.cu:2063-2100):
 * p = 1 / (1 + expf(-l)); selection on p + bias (bias may be NULL), stable (ties -> lower index); weights from
 * the unbiased p; when norm_w: divided by max(double sum, 2^-14); then * w_scale. */
ORC_API int orc_router_sigmoid(const float* logits, const float* bias, int n_tokens, int n_expert, int k, float w_scale,
                               int norm_w, int32_t* ids, float* weights) {
    if (k > n_expert || k > 64) return -1;
    float* p = (float*) malloc(sizeof(float) * (size_t) n_expert);
    float* sel = (float*) malloc(sizeof(float) * (size_t) n_expert);
    uint8_t* taken = (uint8_t*) malloc((size_t) n_expert);
    for (int t = 0; t < n_tokens; ++t) {
        const float* l = logits + (size_t) t * n_expert;
        for (int e = 0; e < n_expert; ++e) {
            p[e] = 1.0f / (1.0f + expf(-l[e]));
            sel[e] = bias ? p[e] + bias[e] : p[e];
            taken[e] = 0;
        }
        double s = 0.0;
        for (int i = 0; i < k; ++i) {
            int bi = -1;
            for (int e = 0; e < n_expert; ++e)
                if (!taken[e] && (bi < 0 || sel[e] > sel[bi])) bi = e;
            taken[bi] = 1;
            ids[(size_t) t * k + i] = bi;
            weights[(size_t) t * k + i] = p[bi];
            s += (double) p[bi];
        }
        for (int i = 0; i < k; ++i) {
            float w = weights[(size_t) t * k + i];
            if (norm_w) w = (float) ((double) w / fmax(s, 6.103515625e-05));
            weights[(size_t) t * k + i] = w * w_scale;
        }
    }
    free(p); free(sel); free(taken);
    return 0;
}

/* ------------------------------------------------------------------ Q8_K activations for the reference's CPU rows
 * ggml's quantize_row_q8_K_ref as the reference transcribes it on the host
 * (quantize_act_parity.cpp:139-176): iscale = -127 / max (the signed value of largest magnitude, first on ties),
 * q = min(127, nearest_int(iscale * x)), bsums per 16, d = 1 / iscale.  292 B / 256. */
static int nearest_int(float f) {
    const float v = f + 12582912.0f;
    int i;
    memcpy(&i, &v, 4);
    return (i & 0x007fffff) - 0x00400000;
}
ORC_API void orc_quantize_q8_K(const float* x, uint8_t* y, int64_t n) {
    memset(y, 0, (size_t) (n / 256) * 292);
    for (int64_t b = 0; b < n / 256; ++b) {
        const float* xb = x + 256 * b;
        uint8_t* o = y + 292 * b;
        float mx = 0.0f, amax = 0.0f;
        for (int j = 0; j < 256; ++j) {
            const float ax = fabsf(xb[j]);
            if (ax > amax) { amax = ax; mx = xb[j]; }
        }
        if (amax == 0.0f) continue;
        const float iscale = -127.0f / mx;
        int8_t* qs = (int8_t*) (o + 4);
        for (int j = 0; j < 256; ++j) {
            const int v = nearest_int(iscale * xb[j]);
            qs[j] = (int8_t) (v < 127 ? v : 127);
        }
        for (int j = 0; j < 16; ++j) {
            int sum = 0;
            for (int i = 0; i < 16; ++i) sum += qs[16 * j + i];
            const int16_t s16 = (int16_t) sum;
            memcpy(o + 4 + 256 + 2 * j, &s16, 2);
        }
        const float d = 1.0f / iscale;
        memcpy(o, &d, 4);
    }
}

/* ------------------------------------------------------------------ in-order cross-rank sum
 * ar_sum_kernel (ds4_kernels.cu:3503-3526): every member adds the members' partials in member order with
 * round-to-nearest adds, so all members hold the same bits.  parts [nm][n]. */
ORC_API void orc_allreduce_in_order(const float* parts, int nm, int64_t n, float* out) {
    for (int64_t i = 0; i < n; ++i) {
        float s = parts[i];
        for (int m = 1; m < nm; ++m) s = s + parts[(size_t) m * n + i];
        out[i] = s;
    }
}

/* ------------------------------------------------------------------ the producer in front of the layer
 * rms_q8_kernel (glm_fast.cu:5669-5697): t = h (+ add); inv = rsqrtf(sum(t^2) / n + eps); x = t * inv * w.  The
 * reference sums the squares in float in an unspecified (tree) order: here the sum is taken in double and rounded once,
 * which every float order matches to a few ulp.  Then the router job of glm_fast_path.cu:6925: logits = router_w . x
 * (float products; summed here in double).  router_w [n_expert][n] as f32. */
ORC_API void orc_rms_router(const float* h, const float* add, const float* w, float eps, int n, const float* router_w,
                            int n_expert, float* h_out, float* x, float* logits) {
    double ss = 0.0;
    for (int e = 0; e < n; ++e) {
        const float t = add ? h[e] + add[e] : h[e];
        if (h_out) h_out[e] = t;
        ss += (double) t * (double) t;
    }
    const float inv = 1.0f / sqrtf((float) ss / (float) n + eps);
    for (int e = 0; e < n; ++e) {
        const float t = add ? h[e] + add[e] : h[e];
        x[e] = t * inv * w[e];
    }
    for (int ex = 0; ex < n_expert; ++ex) {
        double acc = 0.0;
        for (int e = 0; e < n; ++e) acc += (double) router_w[(size_t) ex * n + e] * (double) x[e];
        logits[ex] = (float) acc;
    }
}

/* ------------------------------------------------------------------ hyper-connection write after the FFN block
 * hc_post_kernel (src/kernels/cuda/glm_fast.cu:2747-2757), the consumer of the MoE output: the residual is a stack of 4
 * streams R[s][n_embd]; R_new[d][e] = block_out[e] * post[d] + sum_s comb[d * 4 + s] * R_old[s][e], the sum taken in
 * ascending s as multiply-adds onto the product (the reference's `acc += a * b` compiles to fused multiply-adds). */
ORC_API void orc_hc_post(const float* block_out, const float* R_old, const float* post, const float* comb, int n_embd,
                         float* R_new) {
    for (int d = 0; d < 4; ++d)
        for (int e = 0; e < n_embd; ++e) {
            float acc = block_out[e] * post[d];
            for (int s = 0; s < 4; ++s) acc = fmaf(comb[d * 4 + s], R_old[(size_t) s * n_embd + e], acc);
            R_new[(size_t) d * n_embd + e] = acc;
        }
}

/* ------------------------------------------------------------------ prefill grouping
 * glmb::expert_count / expert_scatter (glm_batch.cu:2102-2133): counts[e]; a stable rank per (token, slot)
 * pair i in ascending i; row = base[id] + rank; row_tok[row] = i / k; pos[i] = row. */
ORC_API void orc_expert_group(const int32_t* ids, int n_pairs, int k, int n_expert, int32_t* counts, int32_t* bounds,
                              int32_t* pos, int32_t* row_tok) {
    for (int e = 0; e < n_expert; ++e) counts[e] = 0;
    for (int i = 0; i < n_pairs; ++i) counts[ids[i]]++;
    bounds[0] = 0;
    for (int e = 0; e < n_expert; ++e) bounds[e + 1] = bounds[e] + counts[e];
    int32_t* fill = (int32_t*) calloc((size_t) n_expert, sizeof(int32_t));
    for (int i = 0; i < n_pairs; ++i) {
        const int e = ids[i], row = bounds[e] + fill[e]++;
        pos[i] = row;
        row_tok[row] = i / k;
    }
    free(fill);
}
