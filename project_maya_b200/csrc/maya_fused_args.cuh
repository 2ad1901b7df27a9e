// maya_fused_args.cuh - the argument block of the single-token layer kernels (moe_fused.cu, moe_stream.cu).
#pragma once

#include "maya_common.cuh"

namespace maya {

struct FusedArgs {
    const float* logits;       // [n_expert]
    int router;                // 0 softmax, 1 sigmoid (+ bias for the selection, weight scale, optional normalisation)
    const float* router_bias;
    float router_w_scale;
    int router_norm_w;
    const float* cpu_part;     // [n_embd] the host lane's contribution, added when *cpu_flag != 0 (NULL: none)
    const int* cpu_flag;
    const void* x;             // [n_embd] f32 or bf16
    int x_is_bf16;
    int n_embd, n_ff, n_expert, k;
    const uint8_t* experts;
    size_t expert_stride;
    int expert_lo, expert_hi;
    const uint8_t* shared;     // NULL: none (or not on this rank)
    int n_ff_sh;
    int sh_lo, sh_hi;          // this rank's slice of the shared expert's FFN width (multiples of 32): its gate/up rows
                               // and the same columns of every down row; the ranks' partial outputs add up
    float limit;
    int* ids;                  // [k] out
    float* weights;            // [k] out
    float* out;                // [n_embd] out
    float* h;                  // scratch [(k + 1)][max(n_ff, n_ff_sh)] f32
    maya_peer_ar ar;           // ar.nm >= 2: sum `out` over the ranks in the epilogue
    int ar_rank;
    unsigned ar_seq;
    maya_hc_post_args hc;      // hc.R_new != NULL: the hyper-connection write of `out` into the residual stack, last
    unsigned* sync;            // scratch: [0] arrivals, [1] epoch, [2] error, [4..13] block 0's phase time stamps (ns)
};

}  // namespace maya
