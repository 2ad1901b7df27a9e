// hc_post.cu - the consumer behind the expert FFN: the hyper-connection write of the block's output into the residual
// stack (4 streams of n_embd floats):  R_new[d][e] = block_out[e] * post[d] + sum_s comb[d * 4 + s] * R_old[s][e].
//
// Reference counterpart: glmf::hc_post (include/strata/kernels/glm_fast.hpp:124, hc_post_kernel,
// src/kernels/cuda/glm_fast.cu:2747-2757, called after the MoE block at src/core/glm_fast_path.cu:7309): one product,
// then four multiply-adds in ascending s - the same operations here, so the bits are the reference's.
//
// The stand-alone launch is for the staged (multi-token) layer paths; for a single token the fused layer kernel does
// this in its epilogue, on the rows each block has just combined (and summed across the ranks): hc_post_rows below.
#include "maya_hc_post.cuh"
#include "maya_internal.cuh"

namespace maya {
namespace {

__global__ void __launch_bounds__(256) hc_post_kernel(const float* __restrict__ block_out, maya_hc_post_args a, int n_embd) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e < n_embd) hc_post_rows(block_out, a, n_embd, e, e + 1, 0, 1);
}

}  // namespace
}  // namespace maya

using namespace maya;

extern "C" int maya_hc_post(const float* block_out, const float* R_old, const float* post, const float* comb, int n_embd,
                            float* R_new, void* stream) {
    if (n_embd <= 0) return MAYA_OK;
    if (!block_out || !R_old || !post || !comb || !R_new) return refuse(MAYA_ERR_ARG);
    if (R_new == R_old) return refuse(MAYA_ERR_ARG);        // every output stream reads all four input streams
    maya_hc_post_args a{R_old, post, comb, R_new};
    hc_post_kernel<<<(n_embd + 255) / 256, 256, 0, as_stream(stream)>>>(block_out, a, n_embd);
    return note_launch("hc_post");
}
