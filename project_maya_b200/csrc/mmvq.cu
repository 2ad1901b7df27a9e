// mmvq.cu - quantized GEMV over GGUF rows: y[c][r] = W_r . x_c for 1..8 q8_1 activation columns.
//
// Replaces native_mmvq (src/kernels/cuda/native_mmvq.cu:1441-1491) and iq_mmvq (src/kernels/cuda/iq_kernels.cu:1015-1036).
// Each warp owns kRowsPerWarp consecutive rows; the activation columns are staged once per block into shared memory
// (structure of arrays, with the integer sums Q4_K needs), every weight call is decoded once and dotted with every
// column, and a column's sum is accumulated in the same order whatever ncols is - so column c of an ncols-wide call
// equals the single-column call bit for bit (the reference's "multi exact" contract, native_mmvq.hpp:25-30).
#include "maya_dots.cuh"

namespace maya {
namespace {

constexpr int kMvWarps = 8;
constexpr int kRowsPerWarp = 2;

template<int T, int NC>
__global__ void __launch_bounds__(kMvWarps * 32) mmvq_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ xq,
                                                             float* __restrict__ y, int n_in, int n_out, int ncols) {
    extern __shared__ __align__(16) uint8_t s_raw[];
    uint32_t* s_tab = (uint32_t*) s_raw;
    int4* xq_q; float* xq_d; int* xq_s;
    const int nblk = n_in / 32;
    const XCols x = xcols_carve(s_raw + Fmt<T>::tab_words * 4, nblk, ncols, &xq_q, &xq_d, &xq_s);
    load_tab<T>(s_tab);
    xcols_stage_p<Dec<T>::xblk, T == MAYA_IQ1_S>(xq, (size_t) nblk * kQ81Bytes, nblk, ncols, xq_q, xq_d, xq_s);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t rb = row_bytes(T, n_in);
    const int r0 = ((int) blockIdx.x * kMvWarps + warp) * kRowsPerWarp;
    if (r0 >= n_out) return;
    const uint8_t* rows[kRowsPerWarp];
#pragma unroll
    for (int j = 0; j < kRowsPerWarp; ++j) rows[j] = w + (size_t) min(r0 + j, n_out - 1) * rb;
    float out[kRowsPerWarp][NC];
    rows_dot<T, kRowsPerWarp, NC>(rows, x, ncols, n_in, lane, s_tab, out);
    if (lane == 0) {
#pragma unroll
        for (int j = 0; j < kRowsPerWarp; ++j)
#pragma unroll
            for (int c = 0; c < NC; ++c)
                if (r0 + j < n_out && c < ncols) y[(size_t) c * n_out + r0 + j] = out[j][c];
    }
}

template<int T, int NC>
int launch_mmvq(const void* w, const void* xq, float* y, int n_in, int n_out, int ncols, cudaStream_t s) {
    const size_t smem = (size_t) Fmt<T>::tab_words * 4 + xcols_bytes(n_in / 32, ncols);
    if (smem > 200 * 1024) return refuse(MAYA_ERR_LIMIT);
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(mmvq_kernel<T, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess)
            return note_launch("mmvq smem attribute");
    }
    const int rows_per_block = kMvWarps * kRowsPerWarp;
    mmvq_kernel<T, NC><<<(n_out + rows_per_block - 1) / rows_per_block, kMvWarps * 32, smem, s>>>(
        (const uint8_t*) w, (const uint8_t*) xq, y, n_in, n_out, ncols);
    return note_launch("mmvq");
}

template<int T>
int launch_mmvq_cols(const void* w, const void* xq, float* y, int n_in, int n_out, int ncols, cudaStream_t s) {
    if (ncols == 1) return launch_mmvq<T, 1>(w, xq, y, n_in, n_out, ncols, s);
    if (ncols == 2) return launch_mmvq<T, 2>(w, xq, y, n_in, n_out, ncols, s);
    if (ncols <= 4) return launch_mmvq<T, 4>(w, xq, y, n_in, n_out, ncols, s);
    return launch_mmvq<T, 8>(w, xq, y, n_in, n_out, ncols, s);
}

}  // namespace
}  // namespace maya

using namespace maya;

extern "C" int maya_mmvq(int type, const void* w, const void* xq, float* y, int n_in, int n_out, int ncols, void* stream) {
    if (!type_qk(type)) return refuse(MAYA_ERR_TYPE);
    if (!w || !xq || !y || n_in <= 0 || n_out <= 0 || n_in % type_qk(type)) return refuse(MAYA_ERR_ARG);
    if (ncols < 1 || ncols > MAYA_MAX_COLS) return refuse(MAYA_ERR_LIMIT);
    if (!aligned16(w) || (((uintptr_t) xq) & 3u)) return refuse(MAYA_ERR_ARG);
    cudaStream_t s = as_stream(stream);
    switch (type) {
        case MAYA_Q8_0: return launch_mmvq_cols<MAYA_Q8_0>(w, xq, y, n_in, n_out, ncols, s);
        case MAYA_Q4_K: return launch_mmvq_cols<MAYA_Q4_K>(w, xq, y, n_in, n_out, ncols, s);
        case MAYA_IQ2_S: return launch_mmvq_cols<MAYA_IQ2_S>(w, xq, y, n_in, n_out, ncols, s);
        case MAYA_IQ3_S: return launch_mmvq_cols<MAYA_IQ3_S>(w, xq, y, n_in, n_out, ncols, s);
        case MAYA_Q5_K: return launch_mmvq_cols<MAYA_Q5_K>(w, xq, y, n_in, n_out, ncols, s);
        case MAYA_Q6_K: return launch_mmvq_cols<MAYA_Q6_K>(w, xq, y, n_in, n_out, ncols, s);
        case MAYA_IQ4_XS: return launch_mmvq_cols<MAYA_IQ4_XS>(w, xq, y, n_in, n_out, ncols, s);
        case MAYA_IQ3_XXS: return launch_mmvq_cols<MAYA_IQ3_XXS>(w, xq, y, n_in, n_out, ncols, s);
        case MAYA_IQ2_XXS: return launch_mmvq_cols<MAYA_IQ2_XXS>(w, xq, y, n_in, n_out, ncols, s);
        default: return launch_mmvq_cols<MAYA_IQ1_S>(w, xq, y, n_in, n_out, ncols, s);
    }
}
