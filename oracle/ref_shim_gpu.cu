// ref_shim_gpu.cu - TEST INFRASTRUCTURE: a C ABI over the reference's own CUDA expert kernels, compiled for sm_100a
// from the reference tree where it lies (oracle/build.py builds this file together with the reference's
// router_top10.cu, iq_kernels.cu, native_mmvq.cu and glm_fast.cu into oracle/_ref/libmaya_ref_gpu.so).
//
// Nothing the library ships links or loads it: the GPU parity tests use it as the live pin (the same blobs, logits and
// activations through the reference's kernels and through this library's), bench.py as "the GPU kernel to beat".
//
// glm_fast.cu refers to four functions of the reference's EXL3 and MLA files that the MoE expert path never calls
// (exl3::mv / set_skip / launch_errors, glmb::mla_decode_v70); they are defined here as stubs so that those files need
// not be built.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <exception>

#include "strata/kernels/exl3.hpp"
#include "strata/kernels/glm_batch.hpp"
#include "strata/kernels/glm_fast.hpp"
#include "strata/kernels/iq_kernels.hpp"
#include "strata/kernels/native_mmvq.hpp"
#include "strata/kernels/router_top10.hpp"

namespace strata::kernels::exl3 {
int launch_errors() { return 0; }
bool mv(const MvJob*, int, cudaStream_t) { return false; }
void set_skip(const int*) {}
}  // namespace strata::kernels::exl3
namespace strata::kernels::glmb {
bool mla_decode_v70(const float*, const uint16_t*, const int*, int, int, int, float, float*, float*, int, cudaStream_t, bool) {
    return false;
}
}  // namespace strata::kernels::glmb

namespace sk = strata::kernels;
namespace gf = strata::kernels::glmf;

#define REF_API extern "C" __attribute__((visibility("default")))

// The calls below may throw (the native_* family) or exit (the oldest kernels); a throw becomes -1.
template<class F> static int guarded(F f) {
    try {
        f();
    } catch (const std::exception& e) {
        std::fprintf(stderr, "reference call threw: %s\n", e.what());
        return -1;
    } catch (...) {
        return -1;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// router_top10 (include/strata/kernels/router_top10.hpp:17)
REF_API int ref_router_top10(const float* logits, int n_tokens, int n_expert, int k, int* ids, float* weights, void* stream) {
    return guarded([&] { sk::router_top10(logits, n_tokens, n_expert, k, ids, weights, stream); });
}
// glmf::quantize_q8_1 (glm_fast.hpp:88)
REF_API int ref_quantize_q8_1(const float* x, void* xq, int n, void* stream) {
    return guarded([&] { gf::quantize_q8_1(x, xq, n, (cudaStream_t) stream); });
}
// quantize_q8_1_rows (iq_kernels.hpp:21)
REF_API int ref_quantize_q8_1_rows(const float* x, int64_t n_rows, int64_t n_cols, void* y, void* stream) {
    return guarded([&] { sk::quantize_q8_1_rows(x, n_rows, n_cols, y, stream); });
}
// iq_mmvq (iq_kernels.hpp:24) and native_mmvq (native_mmvq.hpp:109)
REF_API int ref_iq_mmvq(int type, const void* w, const void* xq, float* y, int n_in, int n_out, int ncols, void* stream) {
    return guarded([&] { sk::iq_mmvq(type, w, xq, y, n_in, n_out, ncols, stream); });
}
REF_API int ref_native_mmvq(int type, const void* w, const void* xq, float* y, int n_in, int n_out, int ncols, void* stream) {
    return guarded([&] { sk::native_mmvq(type, w, xq, y, n_in, n_out, ncols, stream); });
}
REF_API int ref_native_mmvq_supported(int type) { return sk::native_mmvq_supported(type) ? 1 : 0; }
REF_API int ref_iq_supported(int type) { return sk::iq_supported(type) ? 1 : 0; }
REF_API int ref_moe_supported(int type) { return gf::moe_supported(type) ? 1 : 0; }
// glmf::swiglu_q8 (glm_fast.hpp:280)
REF_API int ref_swiglu_q8(const float* gate, const float* up, float limit, int n, void* hq, void* stream) {
    return guarded([&] { gf::swiglu_q8(gate, up, limit, n, hq, (cudaStream_t) stream); });
}

// native_expert_grouped (iq_kernels.hpp:83-92)
REF_API size_t ref_native_expert_scratch_bytes(int64_t cap_entries, int64_t n_ff) {
    return sk::native_expert_scratch_bytes(cap_entries, n_ff);
}
REF_API int ref_native_expert_grouped(int gu_type, int d_type, int64_t n_embd, int64_t n_ff, const unsigned long long* grp_ptr,
                                      const int32_t* grp_start, const int32_t* n_groups, const int32_t* ent_dst,
                                      const int32_t* ent_tok, int64_t cap_groups, int64_t cap_entries, const void* xq,
                                      void* scratch, float* out, void* stream, float limit) {
    int ok = 0;
    const int st = guarded([&] {
        const sk::NativeExpertLayout L = sk::native_expert_layout(gu_type, d_type, n_embd, n_ff);
        ok = sk::native_expert_grouped(L, grp_ptr, grp_start, n_groups, ent_dst, ent_tok, cap_groups, cap_entries, xq, scratch,
                                       out, stream, limit)
                 ? 1 : 0;
    });
    return st != 0 ? st : (ok ? 0 : -3);
}

// glmf::moe_gate_up / moe_down (glm_fast.hpp:496-501): only plan_ptr / plan_w / cpu_part / cpu_flag of MoeDev are read.
// cpu_flag is read unconditionally by moe_down_kernel and moe_win_combine_kernel (glm_fast.cu:5003, 7707): it must be a
// valid device int (one per token for the window), zero when there is no host contribution.
static gf::MoeDev plan_dev(const unsigned long long* plan_ptr, const float* plan_w, const float* cpu_part, const int* cpu_flag) {
    gf::MoeDev d;
    d.plan_ptr = (unsigned long long*) plan_ptr;
    d.plan_w = (float*) plan_w;
    d.cpu_part = (float*) cpu_part;
    d.cpu_flag = (int*) cpu_flag;
    return d;
}
REF_API int ref_moe_gate_up(int gu_type, const unsigned long long* plan_ptr, const float* plan_w, int k, int n_embd, int n_ff,
                            float limit, const void* xq, void* hq, const void* sh_down, int sh_type, const void* sh_hq,
                            int n_ff_sh, float* sh_out, void* stream) {
    return guarded([&] {
        gf::moe_gate_up(gu_type, plan_dev(plan_ptr, plan_w, nullptr, nullptr), k, n_embd, n_ff, limit, xq, hq, sh_down, sh_type,
                        sh_hq, n_ff_sh, sh_out, (cudaStream_t) stream);
    });
}
REF_API int ref_moe_down(int d_type, const unsigned long long* plan_ptr, const float* plan_w, const float* cpu_part,
                         const int* cpu_flag, int k, int n_embd, int n_ff, size_t down_off, const void* hq, const float* sh_out,
                         float* out, void* stream) {
    if (cpu_flag == nullptr) return -4;
    return guarded([&] {
        gf::moe_down(d_type, plan_dev(plan_ptr, plan_w, cpu_part, cpu_flag), k, n_embd, n_ff, down_off, hq, sh_out, out,
                     (cudaStream_t) stream);
    });
}
// glmf::moe_win_experts (glm_fast.hpp:439-465)
REF_API int ref_moe_win_experts(int gu_type, int d_type, const unsigned long long* plan_ptr, const float* plan_w,
                                const float* cpu_part, const int* cpu_flag, const void* xq, size_t xq_stride, void* hq, float* part, const float* sh_out, float* out, size_t out_stride,
                                unsigned long long* grp_ptr, int* grp_start, int* grp_ent, int* n_groups, int T, int k,
                                int n_embd, int n_ff, float limit, size_t down_off, void* stream) {
    if (cpu_flag == nullptr) return -4;
    int ok = 0;
    const int st = guarded([&] {
        gf::MoeWin w;
        w.plan_ptr = plan_ptr; w.plan_w = plan_w; w.cpu_part = cpu_part; w.cpu_flag = cpu_flag; w.xq = xq; w.xq_stride = xq_stride; w.hq = hq; w.part = part;
        w.sh_out = sh_out; w.out = out; w.out_stride = out_stride; w.grp_ptr = grp_ptr; w.grp_start = grp_start;
        w.grp_ent = grp_ent; w.n_groups = n_groups; w.T = T; w.k = k; w.n_embd = n_embd; w.n_ff = n_ff; w.limit = limit;
        w.down_off = down_off;
        ok = gf::moe_win_experts(gu_type, d_type, w, (cudaStream_t) stream) ? 1 : 0;
    });
    return st != 0 ? st : (ok ? 0 : -3);
}
REF_API int ref_launch_errors() { return gf::launch_errors(); }
