// ref_shim_rows.cpp - TEST INFRASTRUCTURE.  C entry points over the reference's own CPU expert rows
// (src/kernels/cpu/iq_avx512.cpp, iq_avx2.cpp; include/strata/kernels/cpu/iq_avx512.hpp:11-17, iq_avx2.hpp:14-20),
// compiled from the reference tree into oracle/_ref/.  Q8_K activations; IQ2_S (22), IQ3_S (21), Q4_K (12).
#include "strata/kernels/cpu/iq_avx2.hpp"
#include "strata/kernels/cpu/iq_avx512.hpp"

#define REF_API extern "C" __attribute__((visibility("default")))
using namespace strata::kernels::cpu;

REF_API int ref_rows_supported(int type, int avx512) { return avx512 ? iq512_supported(type) : iq256_supported(type); }

// ff[t][r] = silu(gate_r . a_t) * (up_r . a_t) for rows [r0, r1)
REF_API void ref_gu_rows(int avx512, int type, const uint8_t* blob, size_t gu_row, size_t up_off, int n,
                         const void* const* act, int nt, float* const* ff, int r0, int r1) {
    if (avx512) iq512_gu_rows(type, blob, gu_row, up_off, n, act, nt, ff, r0, r1);
    else iq256_gu_rows(type, blob, gu_row, up_off, n, act, nt, ff, r0, r1);
}
// out[t][r] = w_r . a_t for rows [r0, r1)
REF_API void ref_rows(int avx512, int type, const uint8_t* w, size_t row_bytes, int n, const void* const* act, int nt,
                      float* const* out, int r0, int r1) {
    if (avx512) iq512_rows(type, w, row_bytes, n, act, nt, out, r0, r1);
    else iq256_rows(type, w, row_bytes, n, act, nt, out, r0, r1);
}
