/*
 * maya_moe.h - C ABI of the B200 (sm_100a) routed-MoE expert-FFN library.
 *
 * One entry point per reference entry point of the path: router -> q8_1 activations -> quantized
 * GEMV (decode) / grouped GEMM (prefill) over unmodified GGUF expert blocks -> weighted combine ->
 * cross-GPU sum.  Plain pointers and sizes only.  Unless a function says otherwise:
 *   - every pointer is a device pointer of the current device; the caller owns all memory, the callee
 *     allocates nothing, never synchronises and enqueues on `stream` (a cudaStream_t; NULL = default
 *     stream, still asynchronous);
 *   - the return value is a status: 0 = enqueued, < 0 = refused (nothing launched), see maya_status;
 *   - ggml type ids: Q8_0 = 8, Q4_K = 12, IQ3_S = 21, IQ2_S = 22;
 *   - weights are unmodified row-major GGUF blocks; expert blob = [gate rows | up rows | down rows];
 *   - blobs, rows and q8_1 buffers must be 16-byte aligned (cudaMalloc gives 256).
 *
 * Each declaration cites the reference interface it replaces (path inside the reference tree : line).
 */
#ifndef MAYA_MOE_H
#define MAYA_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MAYA_API __attribute__((visibility("default")))

enum maya_status {
    MAYA_OK = 0,
    MAYA_ERR_ARG = -1,         /* bad size / null pointer / misalignment */
    MAYA_ERR_TYPE = -2,        /* ggml type without a kernel here */
    MAYA_ERR_LAUNCH = -3,      /* the CUDA launch failed (see maya_last_cuda_error) */
    MAYA_ERR_LIMIT = -4,       /* beyond a documented maximum (k, tokens, experts, scratch) */
    MAYA_ERR_DEVICE = -5       /* not an sm_100 device / no CUDA device */
};

/* ggml type ids.  The first four run on every path (fused single-token kernel, staged decode kernels, window, grouped,
 * prompt-path GEMM).  The others - the rest of glmf::moe_supported's table (glm_fast.cu:5798-5801) that the reference's
 * models use - run on the staged decode paths: maya_mmvq, the plan / window / grouped expert kernels and
 * maya_moe_layer_decode (which then takes its staged kernels); the prompt-path GEMM refuses them. */
enum maya_ggml_type {
    MAYA_Q8_0 = 8, MAYA_Q4_K = 12, MAYA_IQ3_S = 21, MAYA_IQ2_S = 22,
    MAYA_Q5_K = 13, MAYA_Q6_K = 14, MAYA_IQ2_XXS = 16, MAYA_IQ3_XXS = 18, MAYA_IQ1_S = 19, MAYA_IQ4_XS = 23
};

#define MAYA_MAX_K 8            /* plan entries per token (glm_fast.hpp:341) */
#define MAYA_MAX_WIN_TOKENS 16  /* tokens of a window (glm_fast.hpp:459) */
#define MAYA_MAX_COLS 8         /* activation columns of maya_mmvq (native_mmvq.cu:783) */

/* Library / device -------------------------------------------------------------------------------- */
MAYA_API const char* maya_version(void);
/* cudaError_t of the last failed launch on this thread, as an int (0 = none). */
MAYA_API int maya_last_cuda_error(void);
/* Launches refused or failed since load (glmf::launch_errors, glm_fast.cu:5803; mmq::launch_errors, moe_mmq.hpp:99). */
MAYA_API int maya_launch_errors(void);
/* Kernels of this library enqueued successfully since load (every entry point counts its own launches). */
MAYA_API long long maya_launch_count(void);
/* 0 when the current device is sm_100; MAYA_ERR_DEVICE otherwise. */
MAYA_API int maya_device_ok(void);

/* Formats ----------------------------------------------------------------------------------------- */
/* native_mmvq_supported (native_mmvq.hpp:105) / iq_supported (iq_kernels.hpp:17). */
MAYA_API int maya_type_supported(int ggml_type);
/* iq_row_bytes (iq_kernels.hpp:19): bytes of one row of n values; 0 for a bad type or n. */
MAYA_API size_t maya_row_bytes(int ggml_type, int64_t n);
/* native_mmvq_weight_bytes (native_mmvq.hpp:106). */
MAYA_API size_t maya_weight_bytes(int ggml_type, int n_in, int n_out);
/* native_q8_1_bytes (native_mmvq.hpp:30): 36 bytes per 32 values, no row padding. */
MAYA_API size_t maya_q8_1_bytes(int n_in, int ncols);

/* NativeExpertLayout / native_expert_layout (iq_kernels.hpp:63-77). */
typedef struct maya_expert_layout {
    int gu_type, d_type;
    int64_t n_embd, n_ff;
    size_t gu_row, d_row;      /* bytes per row */
    size_t up_off, down_off;   /* byte offsets inside the blob */
    size_t bytes;              /* the whole blob */
    int u_type;                /* the up rows' type (gu_type unless mixed) */
    size_t u_row;
} maya_expert_layout;
MAYA_API int maya_expert_layout_make(int gu_type, int up_type, int d_type, int64_t n_embd, int64_t n_ff,
                                     maya_expert_layout* out);

/* Router ------------------------------------------------------------------------------------------ */
/* router_top10 (router_top10.hpp:17): softmax over all experts (exp and sum in double), stable descending
 * top-k (ties -> lower index), weights renormalised by max(sum, 2^-14).  logits [n_tokens, n_expert] f32;
 * ids [n_tokens, k] i32; weights [n_tokens, k] f32.  k <= 64, n_expert <= 2048.  n_tokens <= 0: no-op, 0. */
MAYA_API int maya_router_top10(const float* logits, int n_tokens, int n_expert, int k, int* ids, float* weights,
                               void* stream);
/* router_sigmoid (router_sigmoid.hpp:27) / glmb::route (glm_batch.hpp:131): p = sigmoid(logit); selection on
 * p + bias (bias NULL: none); weights from the unbiased p, divided by max(sum, 2^-14) when norm_w, times w_scale. */
MAYA_API int maya_router_sigmoid(const float* logits, const float* bias, int n_tokens, int n_expert, int k,
                                 float w_scale, int norm_w, int* ids, float* weights, void* stream);

/* Activations ------------------------------------------------------------------------------------- */
/* native_quantize_q8_1 (native_mmvq.hpp:38) / quantize_q8_1_rows (iq_kernels.hpp:21): x [ncols, n_in] f32 ->
 * ncols * n_in/32 q8_1 blocks {f16 d, f16 sum(x), i8 q[32]}.  n_in % 32 == 0. */
MAYA_API int maya_quantize_q8_1(const float* x, void* x_q8_1, int n_in, int ncols, void* stream);
/* The same from bf16 activations (raw bf16 bits); each value is widened to f32 exactly first. */
MAYA_API int maya_quantize_q8_1_bf16(const uint16_t* x, void* x_q8_1, int n_in, int ncols, void* stream);

/* glmf::swiglu_q8 (glm_fast.hpp:280): h = clamped SwiGLU(gate, up) (limit; INFINITY = plain silu(g) * u), written
 * as n/32 q8_1 blocks.  n % 32 == 0.  The shared expert's h is made with this. */
MAYA_API int maya_swiglu_q8_1(const float* gate, const float* up, float limit, int64_t n, void* hq, void* stream);

/* Quantized GEMV ---------------------------------------------------------------------------------- */
/* native_mmvq (native_mmvq.hpp:109) / iq_mmvq (iq_kernels.hpp:24): y[c * n_out + r] = W_r . x_c, ncols in 1..8;
 * column c's q8_1 blocks at x_q8_1 + c * n_in/32 blocks.  Every column equals its single-column result bit for bit. */
MAYA_API int maya_mmvq(int ggml_type, const void* weights, const void* x_q8_1, float* y, int n_in, int n_out,
                       int ncols, void* stream);

/* Decode experts (plan form) ---------------------------------------------------------------------- */
/* The part of MoeDev the expert kernels read (glm_fast.hpp:293-300): k blob addresses (0 = entry skipped),
 * k router weights, optional CPU-lane partial and flag, optional skip flag (non-zero = do nothing). */
typedef struct maya_moe_plan {
    const unsigned long long* plan_ptr;  /* [k] device addresses of expert blobs */
    const float* plan_w;                 /* [k] */
    const float* cpu_part;               /* [n_embd] or NULL */
    const int* cpu_flag;                 /* [1] or NULL */
    const int* skip;                     /* [1] or NULL */
} maya_moe_plan;

/* glmf::moe_gate_up (glm_fast.hpp:496-498): for each plan entry i < k: rows of gate and up over xq, clamped
 * SwiGLU (limit; INFINITY = unclamped), q8_1 of h into hq[i * n_ff/32 ..].  When sh_down != NULL the same launch
 * computes the shared expert's down rows over sh_hq (n_ff_sh values, type sh_type) into sh_out[n_embd]. */
MAYA_API int maya_moe_gate_up(int gu_type, const maya_moe_plan* plan, int k, int n_embd, int n_ff, float limit,
                              const void* xq, void* hq, const void* sh_down, int sh_type, const void* sh_hq,
                              int n_ff_sh, float* sh_out, void* stream);
/* glmf::moe_down (glm_fast.hpp:499-501): out[r] = sum_i w_i * (down_i[r] . hq_i) in plan order (+ cpu_part[r] when
 * *cpu_flag) + sh_out[r] (when given).  down_off = byte offset of the down rows inside a blob. */
MAYA_API int maya_moe_down(int d_type, const maya_moe_plan* plan, int k, int n_embd, int n_ff, size_t down_off,
                           const void* hq, const float* sh_out, float* out, void* stream);

/* glmf::MoeWin / moe_win_experts (glm_fast.hpp:439-465): T <= 16 tokens, each distinct expert's rows read once for all
 * the tokens that routed it; every token's output equals maya_moe_gate_up + maya_moe_down for it alone, bit for bit. */
typedef struct maya_moe_win {
    const unsigned long long* plan_ptr;  /* [T][8] */
    const float* plan_w;                 /* [T][8] */
    const float* cpu_part;               /* [T][n_embd] or NULL */
    const int* cpu_flag;                 /* [T] or NULL */
    const void* xq;                      /* the tokens' q8_1 inputs, xq_stride bytes apart */
    size_t xq_stride;
    void* hq;                            /* scratch: [T * 8][n_ff / 32] q8_1 */
    float* part;                         /* scratch: [T * 8][n_embd] */
    const float* sh_out;                 /* [T][n_embd] or NULL */
    float* out;                          /* [T][n_embd], out_stride floats apart */
    size_t out_stride;
    unsigned long long* grp_ptr;         /* scratch: [T * 8] */
    int* grp_start;                      /* scratch: [T * 8 + 1] */
    int* grp_ent;                        /* scratch: [T * 8] */
    int* n_groups;                       /* scratch: [1] */
    int T, k, n_embd, n_ff;
    float limit;
    size_t down_off;
} maya_moe_win;
MAYA_API int maya_moe_win_experts(int gu_type, int d_type, const maya_moe_win* w, void* stream);
/* glmf::moe_win_group (glm_fast.hpp:468): the grouping alone. */
MAYA_API int maya_moe_win_group(const maya_moe_win* w, void* stream);

/* Grouped experts (native form) ------------------------------------------------------------------- */
/* native_expert_scratch_bytes (iq_kernels.hpp:80). */
MAYA_API size_t maya_expert_scratch_bytes(int64_t cap_entries, int64_t n_ff);
/* native_expert_grouped (iq_kernels.hpp:89-92): group g's blob at grp_ptr[g]; its entries
 * [grp_start[g], grp_start[g+1]) read token ent_tok[e]'s q8_1 activation and write row ent_dst[e] of out
 * (n_embd floats, unweighted).  *n_groups is read on the device. */
MAYA_API int maya_expert_grouped(const maya_expert_layout* L, const unsigned long long* grp_ptr,
                                 const int32_t* grp_start, const int32_t* n_groups, const int32_t* ent_dst,
                                 const int32_t* ent_tok, int64_t cap_groups, int64_t cap_entries, const void* x_q8_1,
                                 void* scratch, float* out, void* stream, float swiglu_limit);

/* No counterpart in the reference.  maya_expert_grouped for hosts that have no way to hand over scratch memory:
 * an engine whose arena is fully committed to weights and KV cache before the first token, a plug-in running under a
 * framework that owns the allocator, a call site inside a region where cudaMalloc is forbidden.  The q8_1 image of h
 * (the only scratch the grouped path needs) goes into a fixed array inside the library image instead, so this call
 * takes no scratch pointer and performs no allocation of any kind.
 *   - Limit: maya_expert_scratch_bytes(cap_entries, n_ff) must not exceed maya_expert_static_scratch_bytes()
 *     (2 MiB: e.g. 910 entries of FFN width 2048); beyond it the call returns MAYA_ERR_LIMIT, prints why, and
 *     launches nothing.  The array occupies that much memory on every GPU that loads the library, until exit.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current).  Make that first call outside any stream capture.
 *   - All calls share the one array and it keeps whatever the previous call left.  Nothing in it needs clearing: every
 *     entry's slot is written before it is read.  Two calls that may run at the same time on one GPU (different
 *     streams, different host threads) would overwrite each other's h: serialise them. */
MAYA_API size_t maya_expert_static_scratch_bytes(void);
MAYA_API int maya_expert_grouped_static(const maya_expert_layout* L, const unsigned long long* grp_ptr,
                                        const int32_t* grp_start, const int32_t* n_groups, const int32_t* ent_dst,
                                        const int32_t* ent_tok, int64_t cap_groups, int64_t cap_entries,
                                        const void* x_q8_1, float* out, void* stream, float swiglu_limit);

/* Combine ----------------------------------------------------------------------------------------- */
/* native_moe_combine[_multi] (native_moe.hpp:16-20) / moe_combine (shared_expert.hpp:98): per token
 * y = parts[0] * w[0], then fused multiply-adds in expert order, + shared (NULL: none).  parts [n_tok][k][n_embd]. */
MAYA_API int maya_moe_combine(const float* parts, const float* weights, const float* shared, float* y,
                              int64_t n_embd, int64_t k, int n_tok, void* stream);

/* Prefill grouping and glue ------------------------------------------------------------------------ */
/* glmb::expert_count (glm_batch.hpp:133): ids [n] (pair i = token i / k, slot i % k) -> counts[e] and the stable rank
 * of every pair among the pairs of its expert. */
MAYA_API int maya_expert_count(const int* ids, int n, int n_expert, int* counts, int* rank, void* stream);
/* The per-expert bases the reference builds on the host after a device-to-host copy of the counts
 * (src/core/glm_prefill.cu:3239-3255), here on the device: bounds[0] = 0, bounds[e + 1] = bounds[e] + counts[e]. */
MAYA_API int maya_expert_bounds(const int* counts, int n_expert, int* bounds, void* stream);
/* glmb::expert_scatter (glm_batch.hpp:139): row = base[ids[i]] + rank[i]; row_tok[row] = i / k; pos[i] = row. */
MAYA_API int maya_expert_scatter(const int* ids, const int* rank, const int* base, int n, int k, int* row_tok, int* pos,
                                 void* stream);
/* glmb::swiglu_rows (glm_batch.hpp:141): h[r][c] = silu(min(gu[r][c], limit)) * clamp(gu[r][n_ff + c], +-limit) over
 * rows of [gate | up]; ld_h = h's row stride (0: n_ff); h may be gu with ld_h = 2 n_ff. */
MAYA_API int maya_swiglu_rows(const float* gu, float* h, int rows, int n_ff, float limit, int ld_h, void* stream);
/* glmb::moe_combine (glm_batch.hpp:153): ffn[t] = sum_j w[t][j] * out[pos[t * k + j]] + sh[t] (sh NULL: none). */
MAYA_API int maya_moe_combine_rows(const float* out, const int* pos, const float* w, const float* sh, int T, int k,
                                   int n_embd, float* ffn, void* stream);
/* The same for an expert-parallel rank (no counterpart: the reference's prompt path is single-GPU): only the routes
 * whose expert id (ids [T * k]) lies in [e_lo, e_hi) are summed - the other sorted rows were never computed on this
 * rank - so that the ranks' ffn add up to maya_moe_combine_rows' (sh: on one rank only). */
MAYA_API int maya_moe_combine_rows_local(const float* out, const int* pos, const float* w, const int* ids, int e_lo,
                                         int e_hi, const float* sh, int T, int k, int n_embd, float* ffn, void* stream);
/* glmb::moe_combine_add (glm_batch.hpp:150): ffn[t] += sum over the routes of t whose sorted row is in [lo, hi) of
 * w * out[row - base]. */
MAYA_API int maya_moe_combine_add(const float* out, int base, int lo, int hi, const int* pos, const float* w, int T, int k,
                                  int n_embd, float* ffn, void* stream);

/* Prompt-path grouped GEMM on the tensor cores --------------------------------------------------------- */
/* mmq::supported (include/strata/prefill/moe_mmq.hpp:16) / gemm_iq_f16_grouped's iq_supported (iq_kernels.hpp:38-61):
 * types the grouped GEMM takes: Q8_0, Q4_K, IQ2_S, IQ3_S (the i-quants need w_cols % 2048 == 0: 16-byte aligned rows). */
MAYA_API int maya_mmq_supported(int type);
/* mmq::q8_bytes (moe_mmq.hpp:20): bytes of `rows` quantized activation rows of `cols` values.  The rows are stored as
 * f16: each value is d * q of the row's q8_1 rounding as llama.cpp's MMQ quantizer does it (per 32 values
 * d_inv = 127 / amax, q = round(x * d_inv), d = 1 / d_inv, kept as f16), the
 * operand the f16 tensor-core product reads, followed by one f16 per 32 values - f16(sum of the unquantized values)
 * minus the sum of the stored ones, what llama.cpp's MMQ keeps as the "ds4" layout's sum (mmq.cuh:27-46) - padded with
 * zeros to a multiple of 64: (cols + roundup(cols / 32, 64)) * 2 bytes a row.  A Q4_K product multiplies a group's
 * constant term -dmin * m by that sum, as the reference's prompt path does (its decode kernels take the sum of the
 * rounded values instead).  0 for cols % 32 != 0. */
MAYA_API size_t maya_mmq_q8_bytes(int64_t rows, int64_t cols);
/* mmq::quantize (moe_mmq.hpp:34): output row i = the q8_1 image of row ids[i] of x (row i when ids is NULL); x has
 * ld floats a row.  `type` is the weight type the product will use (checked with maya_mmq_supported; the layout is
 * the same for every type). */
MAYA_API int maya_mmq_quantize(const float* x, const int32_t* ids, void* xq, int type, int64_t cols, int64_t ld,
                               int64_t rows, void* stream);
/* The same from bf16 activations (raw bf16 bits, widened to f32 exactly); ld in bf16 elements. */
MAYA_API int maya_mmq_quantize_bf16(const uint16_t* x, const int32_t* ids, void* xq, int type, int64_t cols, int64_t ld,
                                    int64_t rows, void* stream);
/* No counterpart in the reference (which gathers: mmq::quantize with ids = row_tok rounds a token's row once per route):
 * row t of x (tokens rows) is rounded once and its image stored to the k rows pos[t * k + j] of xq (pos as
 * maya_expert_scatter writes it).  xq ends up byte for byte what maya_mmq_quantize(x, row_tok, ...) writes. */
MAYA_API int maya_mmq_quantize_routed(const float* x, const int32_t* pos, int k, void* xq, int type, int64_t cols, int64_t ld,
                                      int64_t tokens, void* stream);
MAYA_API int maya_mmq_quantize_routed_bf16(const uint16_t* x, const int32_t* pos, int k, void* xq, int type, int64_t cols,
                                           int64_t ld, int64_t tokens, void* stream);
/* mmq::Product (moe_mmq.hpp:41-53), field for field, plus three optional fields the reference has no need of. */
typedef struct maya_mmq_product {
    const void* w;               /* n matrices, expert_bytes apart; 16-byte aligned */
    int type;
    int64_t w_rows, w_cols;      /* one matrix: GGUF rows of w_cols values (w_cols % 256 == 0) */
    size_t expert_bytes;         /* a whole number of the type's blocks, a multiple of 16 */
    int n;
    const void* xq;              /* maya_mmq_quantize's output, total_rows rows; 16-byte aligned */
    const int32_t* bounds;       /* device, n + 1 entries (more with expert_map) */
    const int32_t* ids;          /* dst row = ids[row]; NULL: identity */
    int64_t total_rows, max_rows;/* rows of xq; max_rows is not needed here (the grid is sized from total_rows) */
    float* dst;
    int64_t ld_dst;
    const int32_t* expert_map;   /* NULL, or device table: matrix i of w uses bounds[expert_map[i]] (a staged group) */
    unsigned* error;             /* NULL, or device word set to 1 when a bounded wait inside the kernel ran out */
    void* xq_out;                /* maya_mmq_run_glu only, NULL or maya_mmq_q8_bytes(total_rows, n_ff) bytes: h already quantized as
                                    maya_mmq_quantize(h, NULL, ...) would, row = the sorted row (ids not applied);
                                    with it dst may be NULL */
} maya_mmq_product;
/* mmq::Context::run (moe_mmq.hpp:74): for matrix e, rows [bounds[e], bounds[e+1]) of xq times its [w_rows, w_cols]
 * matrix into dst[ids[row]][0 .. w_rows).  w_rows % 128 == 0.  No scratch, no host synchronisation. */
MAYA_API int maya_mmq_run(const maya_mmq_product* p, void* stream);
/* mmq::Context::run_glu (moe_mmq.hpp:81): w_rows = 2 n_ff gate-then-up rows; dst row gets
 * silu(min(gate, limit)) * clamp(up, +-limit) in its first n_ff floats (limit = INFINITY: plain SwiGLU), equal
 * bit for bit to maya_mmq_run followed by maya_swiglu_rows.  n_ff % 128 == 0. */
MAYA_API int maya_mmq_run_glu(const maya_mmq_product* p, float limit, void* stream);

/* The producer in front of the layer: glmf::rms_q8 (glm_fast.hpp:534: h += add; x = rms(h) * norm_w, eps inside the
 * square root) and the router job of the GEMV batch Glm5Model::fast_moe issues next (glm_fast_path.cu:6925:
 * logits = router_w . x, router_w [n_expert][n_embd] F32 or BF16 bits) in ONE launch, so that a decode layer is this call
 * plus maya_moe_layer_decode.  add may be NULL; h_out (the updated residual stream, NULL: not wanted) must not be h when
 * add is given.  x_out is f32 [n_embd]; its q8_1 image is made inside the layer kernel. */
MAYA_API int maya_rms_router(const float* h, const float* add, const float* norm_w, float eps, int n_embd,
                             const void* router_w, int router_is_bf16, int n_expert, float* h_out, float* x_out,
                             float* logits, void* stream);

/* Whole decode layer, one call (no single counterpart: the sequence Glm5Model::fast_moe runs,
 * src/core/glm_fast_path.cu:6917-7100: route -> gate/up -> down + combine, the shared expert alongside). */
typedef struct maya_moe_layer {
    int n_embd, n_ff, n_expert, k;
    int gu_type, d_type;
    const void* experts;         /* n_expert blobs, expert_stride bytes apart */
    size_t expert_stride;
    int n_ff_sh;                 /* 0: no shared expert */
    int sh_gu_type, sh_d_type;
    const void* shared;          /* the shared expert's blob [gate | up | down] */
    float limit;                 /* SwiGLU clamp; INFINITY = none */
    int expert_lo, expert_hi;    /* this rank's experts [lo, hi); others contribute nothing (expert-parallel) */
    int shared_here;             /* non-zero: this rank adds the shared expert */
    int staged;                  /* non-zero: run one token through the staged kernels (router, q8_1, gate/up, down as
                                    separate launches) instead of the single fused kernel; same bits either way */
    int sh_lo, sh_hi;            /* with shared_here: this rank's slice [sh_lo, sh_hi) of the shared expert's FFN width
                                    (multiples of 32; 0, 0 = all of it): its gate/up rows and the same columns of the down
                                    rows, so that the ranks' partial outputs add up to the shared expert's output (the
                                    width-sliced placement; summed in another order than on one rank, so equal to it
                                    only to rounding).  A proper slice needs the single fused kernel (one token, Q8_0
                                    shared expert): otherwise the call is refused */
    int router;                  /* 0: softmax routing (router_top10); 1: sigmoid routing (router_sigmoid.hpp:27,
                                    glmf::moe_route's arithmetic, glm_fast.hpp:426) with the three fields below */
    const float* router_bias;    /* sigmoid: [n_expert] added to the scores for the SELECTION only; NULL: none */
    float router_w_scale;        /* sigmoid: the weights are multiplied by it */
    int router_norm_w;           /* sigmoid: non-zero divides the weights by max(their sum, 2^-14) first */
    const float* cpu_part;       /* the tier hooks of MoeDev (glm_fast.hpp:299-300): [n_tokens][n_embd] - what a host lane */
    const int* cpu_flag;         /* computed for experts that are not resident - added to token t's output when
                                    cpu_flag[t] != 0 (after the routed terms, before the shared expert, moe_down's order);
                                    NULL: no host contribution.  With several ranks give it to one rank only. */
} maya_moe_layer;
/* Bytes of scratch maya_moe_layer_decode needs for n_tokens tokens.  The scratch must be 256-byte aligned and ZEROED
 * once before its first use (it holds the fused kernel's grid-barrier counter); one scratch serves one stream at a
 * time.  After a device-side barrier time-out (a block never arrived) the word returned by maya_moe_layer_error is
 * non-zero and the outputs of that and later calls on the scratch are undefined. */
MAYA_API size_t maya_moe_layer_scratch_bytes(const maya_moe_layer* L, int n_tokens);
/* Reads the sticky barrier-error word of a layer scratch (synchronises the stream first). 0 = no error. */
MAYA_API int maya_moe_layer_error(const maya_moe_layer* L, int n_tokens, const void* scratch, void* stream);
/* Diagnostic: block 0's wall-clock stamps (ns, %globaltimer) of the last fused single-token launch on this scratch:
 * start, end of routing/quantizing, end of its gate/up work, past the grid barrier, end of down + combine, end of the
 * cross-rank sum (= the previous stamp without one).  Synchronises the stream. */
MAYA_API int maya_moe_layer_phase_ns(const maya_moe_layer* L, const void* scratch, void* stream, unsigned long long* out6);
/* logits [n_tokens, n_expert] f32; x [n_tokens, n_embd] f32 (x_is_bf16 == 0) or bf16 bits; out [n_tokens, n_embd] f32;
 * ids / weights [n_tokens, k] (outputs, may be NULL... then scratch holds them).  n_tokens <= MAYA_MAX_WIN_TOKENS. */
MAYA_API int maya_moe_layer_decode(const maya_moe_layer* L, const float* logits, const void* x, int x_is_bf16,
                                   int n_tokens, int* ids, float* weights, float* out, void* scratch,
                                   size_t scratch_bytes, void* stream);

/* Cross-GPU sum of expert partials -------------------------------------------------------------- */
#define MAYA_PEER_AR_MAX_RANKS 8
#define MAYA_PEER_AR_BLOCKS 256        /* flag words per (slot, rank): one per block of the summing kernel */
#define MAYA_PEER_AR_FLAG_STRIDE 32    /* words between flags (128 bytes: one flag per cache line) */

/* PeerArFailure (ds4_kernels.cuh:523-527): written once, by the first wait that ran out. */
typedef struct maya_peer_ar_failure {
    unsigned captured, sequence, observed, block, n4, rank, waited_for, pad;
    unsigned long long elapsed_ns, timeout_ns;
} maya_peer_ar_failure;

/* PeerAr (ds4_kernels.cuh:536-547) for nm ranks.  Every rank owns, in its own HBM, a receive buffer of
 * 2 slots x nm rows x stride floats followed by as many 64-bit {seq, value} words - the form the fused layer kernel
 * exchanges its short rows in, one flagged store per float and no fence - (maya_peer_ar_recv_bytes covers both) and
 * 2 x nm x MAYA_PEER_AR_BLOCKS flags (maya_peer_ar_flag_bytes), all zeroed (flags start at first_seq - 1 = 0, the
 * first call uses seq 1).
 * peer_recv / peer_flags are DEVICE arrays of nm pointers: rank m's buffers as mapped into this rank's address space
 * (peer access or IPC; entry mi = this rank's own).  Calls on each rank's single stream must have matching n and seq,
 * with no skipped calls; seq wraps modulo 2^32.  A wait longer than timeout_ns sets *error (sticky: later calls return
 * at once, leaving x as the local partial); the caller must check it after synchronising.  Not graph-replay safe with a
 * frozen seq. */
typedef struct maya_peer_ar {
    float* recv;
    float* const* peer_recv;
    unsigned* flags;
    unsigned* const* peer_flags;
    unsigned* error;
    maya_peer_ar_failure* failure;   /* optional */
    size_t stride;                   /* floats per row, a multiple of 4, >= n */
    unsigned long long timeout_ns;
    int nm;
    unsigned* seq_counter;           /* optional, TWO device words (zeroed): [0] lets maya_moe_layer_decode_ar and
                                        maya_moe_combine_rows_local_ar take their sequence number from the device (seq
                                        argument 0), so a captured CUDA graph can be replayed; [1] is scratch of those
                                        launches (zero between them) */
} maya_peer_ar;

MAYA_API size_t maya_peer_ar_recv_bytes(int nm, size_t stride);
MAYA_API size_t maya_peer_ar_flag_bytes(int nm);
/* peer_ar_preload (ds4_kernels.cuh:548): loads the kernels on the current device before any rank spins. */
MAYA_API int maya_peer_ar_preload(void* stream);
/* allreduce_peer (ds4_kernels.cuh:546) for nm ranks: x[n] (n % 4 == 0, 16-byte aligned) becomes the sum of the nm
 * ranks' x in rank order - identical bits on every rank. */
MAYA_API int maya_allreduce_peer(float* x, int n, const maya_peer_ar* a, int mi, unsigned seq, void* stream);
/* maya_moe_layer_decode followed by that sum of `out` over the ranks.  One token: the sum runs in the epilogue of the
 * fused layer kernel (each block pushes the output rows it just combined to every peer, then adds the peers' rows in rank
 * order) - no separate launch.  2..16 tokens: the window kernels, the sum inside their last launch: the combine kernel's
 * blocks exchange the rows they have just combined (the reference runs a separate allreduce over out[T * n_embd] after
 * win_experts, src/ds4/ds4_model.cu:22822-22828).
 * seq == 0: the kernel uses *a->seq_counter + 1 and stores it back when it ends, so every rank's n-th call carries n
 * without the host counting - the form to capture in a CUDA graph (a single token through the staged kernels excepted). */
MAYA_API int maya_moe_layer_decode_ar(const maya_moe_layer* L, const float* logits, const void* x, int x_is_bf16,
                                      int n_tokens, int* ids, float* weights, float* out, void* scratch,
                                      size_t scratch_bytes, const maya_peer_ar* a, int mi, unsigned seq, void* stream);
/* The prompt path's last step on an expert-parallel rank, with the cross-rank sum in the same launch:
 * maya_moe_combine_rows_local into ffn [T][n_embd] (contiguous, 16-byte aligned, T * n_embd <= a->stride), each block then
 * exchanging the rows it has combined - ffn ends as the rank-ordered sum over the nm ranks, the same bits on every rank.
 * No counterpart (the reference's prompt path is single-GPU; its decode path sums with a separate allreduce launch). */
MAYA_API int maya_moe_combine_rows_local_ar(const float* out, const int* pos, const float* w, const int* ids, int e_lo,
                                            int e_hi, const float* sh, int T, int k, int n_embd, float* ffn,
                                            const maya_peer_ar* a, int mi, unsigned seq, void* stream);
/* The consumer behind the block: glmf::hc_post (include/strata/kernels/glm_fast.hpp:124; hc_post_kernel,
 * src/kernels/cuda/glm_fast.cu:2747-2757).  The residual is a stack of 4 streams of n_embd floats;
 * R_new[d][e] = block_out[e] * post[d] + sum_s comb[d * 4 + s] * R_old[s][e] (post[4], comb[16] dst-major, device
 * memory).  R_new must not alias R_old. */
typedef struct maya_hc_post_args {
    const float* R_old;   /* [4][n_embd] */
    const float* post;    /* [4] */
    const float* comb;    /* [4][4]: comb[d * 4 + s] weighs input stream s in output stream d */
    float* R_new;         /* [4][n_embd] */
} maya_hc_post_args;
MAYA_API int maya_hc_post(const float* block_out, const float* R_old, const float* post, const float* comb, int n_embd,
                          float* R_new, void* stream);
/* maya_moe_layer_decode[_ar] followed by that write, one token (n_tokens tokens: hc points to n_tokens structures' worth
 * of arrays, token t at R_old + t * 4 * n_embd, post + t * 4, comb + t * 16, R_new + t * 4 * n_embd).  `a` may be NULL
 * (one rank: no cross-rank sum).  One token: the write happens in the fused layer kernel's epilogue, each block on the
 * output rows it has just combined and summed - what Glm5Model::fast_moe follows the block with
 * (src/core/glm_fast_path.cu:7309) costs no launch.  `out` still receives the block's output. */
MAYA_API int maya_moe_layer_decode_hc(const maya_moe_layer* L, const float* logits, const void* x, int x_is_bf16,
                                      int n_tokens, int* ids, float* weights, float* out, void* scratch,
                                      size_t scratch_bytes, const maya_peer_ar* a, int mi, unsigned seq,
                                      const maya_hc_post_args* hc, void* stream);
/* Set-up helpers (startup only, they allocate and synchronise): a zeroed device buffer another process on the same
 * machine can map. */
MAYA_API int maya_peer_buffer_create(size_t bytes, void** ptr, unsigned char handle[64]);
MAYA_API int maya_peer_buffer_open(const unsigned char handle[64], void** ptr);
MAYA_API int maya_peer_buffer_close(void* ptr);
MAYA_API int maya_peer_buffer_destroy(void* ptr);

/* Synthetic expert weights (bench / test support; host-callable generators) ------------------------ */
/* Quantize rows of f32 weights to a GGUF type (own quantizers: nearest-codeword search for the i-quants).
 * Host memory in, host memory out.  n_cols a multiple of the block size. */
MAYA_API int maya_quantize_weights_host(int ggml_type, const float* w, int64_t n_rows, int64_t n_cols, void* out);
/* The same on the device, the weights drawn N(0, sigma) from a counter-based generator keyed by (seed, index):
 * fills n_rows * n_cols values' worth of blocks at `out` (device). */
MAYA_API int maya_synth_weights(int ggml_type, uint64_t seed, float sigma, int64_t n_rows, int64_t n_cols, void* out,
                                void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MAYA_MOE_H */
