// moe_layer.cu - one decode MoE layer in one call: route -> q8_1(x) -> routed gate/up + SwiGLU -> down + combine,
// the always-on shared expert alongside.  The sequence Glm5Model::fast_moe drives in the reference
// (src/core/glm_fast_path.cu:6917-7100), without the tier plan: every expert is resident, the plan of a token is the
// blob addresses of its k routed experts (0 for experts outside [expert_lo, expert_hi): another rank's).
#include <math.h>

#include "maya_internal.cuh"

namespace maya {
namespace {

struct Scratch {
    uint8_t* xq;                 // [T][n_embd/32] q8_1
    unsigned long long* plan_ptr;  // [T][8]
    float* plan_w;               // [T][8]
    int* ids;                    // [T][k]
    float* weights;              // [T][k]
    uint8_t* hq;                 // [T*8][n_ff/32] q8_1
    float* part;                 // [T*8][n_embd]      (T > 1)
    unsigned long long* grp_ptr; // [T*8]
    int* grp_start;              // [T*8 + 1]
    int* grp_ent;                // [T*8]
    int* n_groups;               // [1]
    float* sh_gu;                // [T][2 * n_ff_sh]
    uint8_t* sh_hq;              // [T][n_ff_sh/32] q8_1
    float* sh_out;               // [T][n_embd]
    float* h;                    // the fused single-token kernel's h: q8_1 image, shared-unit halves, counters
    unsigned* sync;              // [16]: the fused kernel's barrier counter, epoch, error word (zero before first use)
    size_t bytes;
};

size_t align_up(size_t v) { return (v + 255) & ~(size_t) 255; }

Scratch carve(const maya_moe_layer& L, int T, uint8_t* base) {
    Scratch s{};
    size_t off = 0;
    auto take = [&](size_t n) { uint8_t* p = base ? base + off : nullptr; off += align_up(n); return p; };
    // the fused kernel's words first: their place must not depend on T (a scratch sized for a window also serves
    // single tokens, and the barrier counter has to survive the calls in between)
    s.sync = (unsigned*) take(16 * sizeof(unsigned));
    {
        const int ld = L.n_ff > L.n_ff_sh ? L.n_ff : L.n_ff_sh;
        // per expert and 32-value group of h: the q8_1 image (40 bytes), the f32 halves two blocks leave when a unit is
        // shared between them (128 bytes) and that unit's arrival counter
        s.h = (float*) take((size_t) (MAYA_MAX_K + 1) * (ld / 32) * (40 + 128 + 4));
    }
    s.xq = take((size_t) T * (L.n_embd / 32) * kQ81Bytes);
    s.plan_ptr = (unsigned long long*) take((size_t) T * 8 * sizeof(unsigned long long));
    s.plan_w = (float*) take((size_t) T * 8 * sizeof(float));
    s.ids = (int*) take((size_t) T * L.k * sizeof(int));
    s.weights = (float*) take((size_t) T * L.k * sizeof(float));
    s.hq = take((size_t) T * 8 * (L.n_ff / 32) * kQ81Bytes);
    s.part = (float*) take(T > 1 ? (size_t) T * 8 * L.n_embd * sizeof(float) : 0);
    s.grp_ptr = (unsigned long long*) take((size_t) T * 8 * sizeof(unsigned long long));
    s.grp_start = (int*) take(((size_t) T * 8 + 1) * sizeof(int));
    s.grp_ent = (int*) take((size_t) T * 8 * sizeof(int));
    s.n_groups = (int*) take(sizeof(int));
    if (L.n_ff_sh > 0) {
        s.sh_gu = (float*) take((size_t) T * 2 * L.n_ff_sh * sizeof(float));
        s.sh_hq = take((size_t) T * (L.n_ff_sh / 32) * kQ81Bytes);
        s.sh_out = (float*) take((size_t) T * L.n_embd * sizeof(float));
    }
    s.bytes = off;
    return s;
}

__global__ void plan_kernel(const int* __restrict__ ids, const float* __restrict__ weights, int T, int k,
                            const uint8_t* experts, size_t stride, int lo, int hi,
                            unsigned long long* __restrict__ plan_ptr, float* __restrict__ plan_w) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * 8) return;
    const int t = i >> 3, j = i & 7;
    unsigned long long p = 0ull;
    float w = 0.0f;
    if (j < k) {
        const int e = ids[t * k + j];
        w = weights[t * k + j];
        if (e >= lo && e < hi) p = (unsigned long long) (experts + (size_t) e * stride);
    }
    plan_ptr[i] = p;
    plan_w[i] = w;
}

int check_layer(const maya_moe_layer* L) {
    if (!L || !L->experts) return MAYA_ERR_ARG;
    if (!type_qk(L->gu_type) || !type_qk(L->d_type)) return MAYA_ERR_TYPE;
    if (L->k < 1 || L->k > MAYA_MAX_K || L->n_expert < L->k) return MAYA_ERR_LIMIT;
    if (L->n_embd <= 0 || L->n_ff <= 0 || L->n_embd % type_qk(L->gu_type) || L->n_ff % type_qk(L->d_type) || L->n_ff % 32 ||
        L->n_embd % 32)
        return MAYA_ERR_ARG;
    if (L->n_ff_sh > 0) {
        if (!L->shared) return MAYA_ERR_ARG;
        if (!type_is_core(L->sh_gu_type) || !type_is_core(L->sh_d_type)) return MAYA_ERR_TYPE;
        if (L->n_embd % type_qk(L->sh_gu_type) || L->n_ff_sh % type_qk(L->sh_d_type) || L->n_ff_sh % 32) return MAYA_ERR_ARG;
    }
    if (L->expert_lo < 0 || L->expert_hi > L->n_expert || L->expert_lo > L->expert_hi) return MAYA_ERR_ARG;
    if (L->router != 0 && L->router != 1) return MAYA_ERR_ARG;
    if (L->cpu_flag != nullptr && L->cpu_part == nullptr) return MAYA_ERR_ARG;
    if (L->sh_lo != 0 || L->sh_hi != 0) {            // a slice of the shared expert's width
        if (L->sh_lo < 0 || L->sh_hi > L->n_ff_sh || L->sh_lo > L->sh_hi || L->sh_lo % 32 || L->sh_hi % 32) return MAYA_ERR_ARG;
    }
    return MAYA_OK;
}

}  // namespace
}  // namespace maya

using namespace maya;

extern "C" size_t maya_moe_layer_scratch_bytes(const maya_moe_layer* L, int n_tokens) {
    if (check_layer(L) != MAYA_OK || n_tokens < 1 || n_tokens > MAYA_MAX_WIN_TOKENS) return 0;
    return carve(*L, n_tokens, nullptr).bytes;
}

extern "C" int maya_moe_layer_error(const maya_moe_layer* L, int n_tokens, const void* scratch, void* stream) {
    if (check_layer(L) != MAYA_OK || !scratch || n_tokens < 1 || n_tokens > MAYA_MAX_WIN_TOKENS) return MAYA_ERR_ARG;
    const Scratch S = carve(*L, n_tokens, (uint8_t*) scratch);
    unsigned word = 0;
    if (cudaStreamSynchronize(as_stream(stream)) != cudaSuccess) return note_launch("layer_error sync");
    if (cudaMemcpy(&word, S.sync + 2, sizeof(word), cudaMemcpyDeviceToHost) != cudaSuccess) return note_launch("layer_error copy");
    return (int) word;
}

extern "C" int maya_moe_layer_phase_ns(const maya_moe_layer* L, const void* scratch, void* stream, unsigned long long* out6) {
    if (check_layer(L) != MAYA_OK || !scratch || !out6) return MAYA_ERR_ARG;
    const Scratch S = carve(*L, 1, (uint8_t*) scratch);
    if (cudaStreamSynchronize(as_stream(stream)) != cudaSuccess) return note_launch("phase_ns sync");
    if (cudaMemcpy(out6, S.sync + 4, 6 * sizeof(unsigned long long), cudaMemcpyDeviceToHost) != cudaSuccess)
        return note_launch("phase_ns copy");
    return MAYA_OK;
}

static int layer_decode(const maya_moe_layer* L, const float* logits, const void* x, int x_is_bf16, int n_tokens, int* ids,
                        float* weights, float* out, void* scratch, size_t scratch_bytes, const maya_peer_ar* ar, int mi,
                        unsigned seq, void* stream, const maya_hc_post_args* hc = nullptr);
static int ar_args_ok(const maya_moe_layer* L, int n_tokens, float* out, const maya_peer_ar* a, int mi, unsigned seq);

extern "C" int maya_moe_layer_decode(const maya_moe_layer* L, const float* logits, const void* x, int x_is_bf16,
                                     int n_tokens, int* ids, float* weights, float* out, void* scratch,
                                     size_t scratch_bytes, void* stream) {
    return layer_decode(L, logits, x, x_is_bf16, n_tokens, ids, weights, out, scratch, scratch_bytes, nullptr, 0, 0, stream);
}

extern "C" int maya_moe_layer_decode_ar(const maya_moe_layer* L, const float* logits, const void* x, int x_is_bf16,
                                        int n_tokens, int* ids, float* weights, float* out, void* scratch,
                                        size_t scratch_bytes, const maya_peer_ar* a, int mi, unsigned seq, void* stream) {
    if (ar_args_ok(L, n_tokens, out, a, mi, seq) != MAYA_OK) return refuse(MAYA_ERR_ARG);
    return layer_decode(L, logits, x, x_is_bf16, n_tokens, ids, weights, out, scratch, scratch_bytes, a, mi, seq, stream);
}

static int ar_args_ok(const maya_moe_layer* L, int n_tokens, float* out, const maya_peer_ar* a, int mi, unsigned seq) {
    if (!a || a->nm < 2 || a->nm > MAYA_PEER_AR_MAX_RANKS || mi < 0 || mi >= a->nm || !a->recv || !a->peer_recv ||
        !a->flags || !a->peer_flags || !a->error || a->timeout_ns == 0 || a->stride % 4)
        return MAYA_ERR_ARG;
    if (L && n_tokens > 0 && (size_t) n_tokens * L->n_embd > a->stride) return MAYA_ERR_ARG;
    if (out && !aligned16(out)) return MAYA_ERR_ARG;
    // the device-side sequence number lives in the fused single-token kernel and in the window's combine launch
    if (seq == 0u && (a->seq_counter == nullptr || (n_tokens == 1 && L && (L->staged || !fused_t1_supported(*L)))))
        return MAYA_ERR_ARG;
    return MAYA_OK;
}

extern "C" int maya_moe_layer_decode_hc(const maya_moe_layer* L, const float* logits, const void* x, int x_is_bf16,
                                        int n_tokens, int* ids, float* weights, float* out, void* scratch,
                                        size_t scratch_bytes, const maya_peer_ar* a, int mi, unsigned seq,
                                        const maya_hc_post_args* hc, void* stream) {
    if (!hc || !hc->R_old || !hc->post || !hc->comb || !hc->R_new || hc->R_new == hc->R_old) return refuse(MAYA_ERR_ARG);
    if (a != nullptr && ar_args_ok(L, n_tokens, out, a, mi, seq) != MAYA_OK) return refuse(MAYA_ERR_ARG);
    return layer_decode(L, logits, x, x_is_bf16, n_tokens, ids, weights, out, scratch, scratch_bytes, a, mi, seq, stream, hc);
}

// The staged paths' consumer: one hc_post launch per token, after `out` is complete.
static int hc_post_tokens(const maya_hc_post_args* hc, const float* out, int T, int n_embd, void* stream) {
    if (hc == nullptr) return MAYA_OK;
    for (int t = 0; t < T; ++t) {
        const int st = maya_hc_post(out + (size_t) t * n_embd, hc->R_old + (size_t) t * 4 * n_embd, hc->post + t * 4,
                                    hc->comb + t * 16, n_embd, hc->R_new + (size_t) t * 4 * n_embd, stream);
        if (st != MAYA_OK) return st;
    }
    return MAYA_OK;
}

static int layer_decode(const maya_moe_layer* L, const float* logits, const void* x, int x_is_bf16, int n_tokens, int* ids,
                        float* weights, float* out, void* scratch, size_t scratch_bytes, const maya_peer_ar* ar, int mi,
                        unsigned seq, void* stream, const maya_hc_post_args* hc) {
    int st = check_layer(L);
    if (st != MAYA_OK) return refuse(st);
    if (n_tokens < 1 || n_tokens > MAYA_MAX_WIN_TOKENS) return refuse(MAYA_ERR_LIMIT);
    if (!logits || !x || !out || !scratch || (((uintptr_t) scratch) & 255u)) return refuse(MAYA_ERR_ARG);
    const int T = n_tokens;
    const Scratch S = carve(*L, T, (uint8_t*) scratch);
    if (S.bytes > scratch_bytes) return refuse(MAYA_ERR_LIMIT);
    cudaStream_t s = as_stream(stream);
    int* d_ids = ids ? ids : S.ids;
    float* d_w = weights ? weights : S.weights;
    if (T == 1 && !L->staged && fused_t1_supported(*L))
        return fused_t1(*L, logits, x, x_is_bf16, d_ids, d_w, out, S.h, S.sync, ar, mi, seq, hc, s);
    if (L->n_ff_sh > 0 && L->shared_here && (L->sh_lo != 0 || (L->sh_hi != 0 && L->sh_hi != L->n_ff_sh)))
        return refuse(MAYA_ERR_ARG);                 // only the fused kernel slices the shared expert

    st = L->router == 1 ? maya_router_sigmoid(logits, L->router_bias, T, L->n_expert, L->k, L->router_w_scale, L->router_norm_w,
                                              d_ids, d_w, stream)
                        : maya_router_top10(logits, T, L->n_expert, L->k, d_ids, d_w, stream);
    if (st != MAYA_OK) return st;
    st = x_is_bf16 ? maya_quantize_q8_1_bf16((const uint16_t*) x, S.xq, L->n_embd, T, stream)
                   : maya_quantize_q8_1((const float*) x, S.xq, L->n_embd, T, stream);
    if (st != MAYA_OK) return st;
    plan_kernel<<<(T * 8 + 127) / 128, 128, 0, s>>>(d_ids, d_w, T, L->k, (const uint8_t*) L->experts, L->expert_stride,
                                                    L->expert_lo, L->expert_hi, S.plan_ptr, S.plan_w);
    st = note_launch("moe_plan");
    if (st != MAYA_OK) return st;

    const bool shared = L->n_ff_sh > 0 && L->shared_here;
    const uint8_t* sh_blob = (const uint8_t*) L->shared;
    size_t sh_down_off = 0;
    if (shared) {
        sh_down_off = row_bytes(L->sh_gu_type, L->n_embd) * (size_t) L->n_ff_sh * 2;
        for (int c0 = 0; c0 < T; c0 += MAYA_MAX_COLS) {   // gate and up rows are contiguous: one GEMV of 2 * n_ff_sh rows
            const int nc = T - c0 < MAYA_MAX_COLS ? T - c0 : MAYA_MAX_COLS;
            // column-major output [c][2 * n_ff_sh] per call: offset by the columns already done
            st = maya_mmvq(L->sh_gu_type, sh_blob, S.xq + (size_t) c0 * (L->n_embd / 32) * kQ81Bytes,
                           S.sh_gu + (size_t) c0 * 2 * L->n_ff_sh, L->n_embd, 2 * L->n_ff_sh, nc, stream);
            if (st != MAYA_OK) return st;
        }
        for (int c = 0; c < T; ++c) {
            st = maya_swiglu_q8_1(S.sh_gu + (size_t) c * 2 * L->n_ff_sh, S.sh_gu + (size_t) c * 2 * L->n_ff_sh + L->n_ff_sh,
                                  L->limit, L->n_ff_sh, S.sh_hq + (size_t) c * (L->n_ff_sh / 32) * kQ81Bytes, stream);
            if (st != MAYA_OK) return st;
        }
    }

    const size_t up_off = row_bytes(L->gu_type, L->n_embd) * (size_t) L->n_ff;
    const size_t down_off = 2 * up_off;
    if (T == 1) {
        maya_moe_plan P{S.plan_ptr, S.plan_w, L->cpu_flag ? L->cpu_part : nullptr, L->cpu_flag, nullptr};
        st = maya_moe_gate_up(L->gu_type, &P, L->k, L->n_embd, L->n_ff, L->limit, S.xq, S.hq,
                              shared ? sh_blob + sh_down_off : nullptr, L->sh_d_type, S.sh_hq, L->n_ff_sh, S.sh_out, stream);
        if (st != MAYA_OK) return st;
        st = maya_moe_down(L->d_type, &P, L->k, L->n_embd, L->n_ff, down_off, S.hq, shared ? S.sh_out : nullptr, out, stream);
        if (st == MAYA_OK && ar != nullptr) st = maya_allreduce_peer(out, L->n_embd, ar, mi, seq, stream);
        return st == MAYA_OK ? hc_post_tokens(hc, out, 1, L->n_embd, stream) : st;
    }
    if (shared) {
        for (int c0 = 0; c0 < T; c0 += MAYA_MAX_COLS) {
            const int nc = T - c0 < MAYA_MAX_COLS ? T - c0 : MAYA_MAX_COLS;
            st = maya_mmvq(L->sh_d_type, sh_blob + sh_down_off, S.sh_hq + (size_t) c0 * (L->n_ff_sh / 32) * kQ81Bytes,
                           S.sh_out + (size_t) c0 * L->n_embd, L->n_ff_sh, L->n_embd, nc, stream);
            if (st != MAYA_OK) return st;
        }
    }
    maya_moe_win W{};
    W.plan_ptr = S.plan_ptr;
    W.plan_w = S.plan_w;
    W.xq = S.xq;
    W.xq_stride = (size_t) (L->n_embd / 32) * kQ81Bytes;
    W.hq = S.hq;
    W.part = S.part;
    W.cpu_part = L->cpu_flag ? L->cpu_part : nullptr;
    W.cpu_flag = L->cpu_flag;
    W.sh_out = shared ? S.sh_out : nullptr;
    W.out = out;
    W.out_stride = (size_t) L->n_embd;
    W.grp_ptr = S.grp_ptr;
    W.grp_start = S.grp_start;
    W.grp_ent = S.grp_ent;
    W.n_groups = S.n_groups;
    W.T = T;
    W.k = L->k;
    W.n_embd = L->n_embd;
    W.n_ff = L->n_ff;
    W.limit = L->limit;
    W.down_off = down_off;
    st = win_experts(L->gu_type, L->d_type, &W, ar, mi, seq, s);       // with `ar`: the sum runs in the combine launch
    return st == MAYA_OK ? hc_post_tokens(hc, out, T, L->n_embd, stream) : st;
}
