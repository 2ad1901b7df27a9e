// maya_internal.cuh - host-side entry points shared between translation units of the library.
#pragma once

#include "maya_common.cuh"

namespace maya {

// How the group kernels find their work: group g = blob ptr[g] with entries [start[g], start[g+1]) (start NULL: the
// single entry g).  Entry e has an h / partial slot (ent_slot[e], NULL: e), an activation column (ent_tok[e]; NULL:
// slot >> 3 when tok_from_slot, else 0) and an output row for the down product (ent_out[e], NULL: its slot).
struct GroupArgs {
    const unsigned long long* ptr;
    const int* start;
    const int* n_groups;
    const int* ent_slot;
    const int* ent_tok;
    const int* ent_out;
    const int* skip;
    int tok_from_slot;
    int cap_entries;      // > 0: the kernels touch no entry at or beyond it
};

int gate_up_groups(int gu_type, const GroupArgs& A, int n_groups_grid, int n_embd, int n_ff, size_t up_off, float limit,
                   const void* xq, size_t xq_stride, void* hq, const void* sh_down, int sh_type, const void* sh_hq,
                   int n_ff_sh, float* sh_out, cudaStream_t s);
int down_groups(int d_type, const GroupArgs& A, int n_groups_grid, int n_embd, int n_ff, size_t down_off, const void* hq,
                float* part, cudaStream_t s);
int down_plan(int d_type, const maya_moe_plan& P, int k, int n_embd, int n_ff, size_t down_off, const void* hq,
              const float* sh_out, float* out, cudaStream_t s);
int win_combine(const unsigned long long* plan_ptr, const float* plan_w, int T, int k, int n_embd, const float* part,
                const float* cpu_part, const int* cpu_flag, const float* sh_out, float* out, size_t out_stride,
                cudaStream_t s);

int win_experts(int gu_type, int d_type, const maya_moe_win* w, const maya_peer_ar* ar, int mi, unsigned seq, cudaStream_t s);

// The fused single-token layer kernel (moe_fused.cu).
bool fused_t1_supported(const maya_moe_layer& L);
int fused_t1(const maya_moe_layer& L, const float* logits, const void* x, int x_is_bf16, int* ids, float* weights,
             float* out, float* h_scratch, unsigned* sync, const maya_peer_ar* ar, int ar_rank, unsigned ar_seq,
             const maya_hc_post_args* hc, cudaStream_t s);

}  // namespace maya
