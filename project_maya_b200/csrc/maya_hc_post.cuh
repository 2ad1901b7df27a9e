// maya_hc_post.cuh - the hyper-connection write's arithmetic, shared by the stand-alone kernel (hc_post.cu) and the
// fused layer kernel's epilogue (moe_fused.cu).
#pragma once

#include "maya_common.cuh"

namespace maya {

// Elements [e0, e1) of all four output streams, by threads tid, tid + nt, ...:
// acc = block_out[e] * post[d]; acc = fma(comb[d * 4 + s], R_old[s][e], acc) for s = 0..3 (hc_post_kernel's order).
__device__ __forceinline__ void hc_post_rows(const float* block_out, const maya_hc_post_args& a, int n_embd, int e0, int e1,
                                             int tid, int nt) {
    for (int e = e0 + tid; e < e1; e += nt) {
        const float b = block_out[e];
        float r[4];
#pragma unroll
        for (int s = 0; s < 4; ++s) r[s] = a.R_old[(size_t) s * n_embd + e];
#pragma unroll
        for (int d = 0; d < 4; ++d) {
            float acc = __fmul_rn(b, a.post[d]);
#pragma unroll
            for (int s = 0; s < 4; ++s) acc = __fmaf_rn(a.comb[d * 4 + s], r[s], acc);
            a.R_new[(size_t) d * n_embd + e] = acc;
        }
    }
}

}  // namespace maya
