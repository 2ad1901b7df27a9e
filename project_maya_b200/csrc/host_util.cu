// host_util.cu - status bookkeeping and format/layout helpers.
#include <atomic>
#include <cstdio>

#include "maya_common.cuh"

namespace maya {

static std::atomic<int> g_launch_errors{0};
static std::atomic<long long> g_launches{0};
static thread_local int t_last_cuda_error = 0;

int note_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) { g_launches.fetch_add(1, std::memory_order_relaxed); return MAYA_OK; }
    t_last_cuda_error = (int) e;
    if (g_launch_errors.fetch_add(1) < 8) std::fprintf(stderr, "maya_moe: %s: %s\n", what, cudaGetErrorString(e));
    return MAYA_ERR_LAUNCH;
}
int refuse(int status) {
    g_launch_errors.fetch_add(1);
    return status;
}

}  // namespace maya

using namespace maya;

extern "C" {

const char* maya_version(void) { return "maya-moe-b200 0.1 (sm_100a)"; }
int maya_last_cuda_error(void) { return t_last_cuda_error; }
int maya_launch_errors(void) { return g_launch_errors.load(); }
long long maya_launch_count(void) { return g_launches.load(); }

int maya_device_ok(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return MAYA_ERR_DEVICE; }
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
        cudaGetLastError();
        return MAYA_ERR_DEVICE;
    }
    return major == 10 ? MAYA_OK : MAYA_ERR_DEVICE;
}

int maya_type_supported(int t) { return type_qk(t) != 0; }
size_t maya_row_bytes(int t, int64_t n) {
    const int q = type_qk(t);
    if (!q || n <= 0 || n % q) return 0;
    return row_bytes(t, n);
}
size_t maya_weight_bytes(int t, int n_in, int n_out) {
    if (n_out <= 0) return 0;
    return maya_row_bytes(t, n_in) * (size_t) n_out;
}
size_t maya_q8_1_bytes(int n_in, int ncols) {
    if (n_in <= 0 || n_in % 32 || ncols <= 0) return 0;
    return (size_t) (n_in / 32) * kQ81Bytes * (size_t) ncols;
}

int maya_expert_layout_make(int gu_type, int up_type, int d_type, int64_t n_embd, int64_t n_ff, maya_expert_layout* L) {
    if (!L) return MAYA_ERR_ARG;
    if (!type_qk(gu_type) || !type_qk(up_type) || !type_qk(d_type)) return MAYA_ERR_TYPE;
    if (n_embd <= 0 || n_ff <= 0 || n_embd % type_qk(gu_type) || n_embd % type_qk(up_type) || n_ff % type_qk(d_type) ||
        n_ff % 32)
        return MAYA_ERR_ARG;
    L->gu_type = gu_type;
    L->u_type = up_type;
    L->d_type = d_type;
    L->n_embd = n_embd;
    L->n_ff = n_ff;
    L->gu_row = row_bytes(gu_type, n_embd);
    L->u_row = row_bytes(up_type, n_embd);
    L->d_row = row_bytes(d_type, n_ff);
    L->up_off = L->gu_row * (size_t) n_ff;
    L->down_off = L->up_off + L->u_row * (size_t) n_ff;
    L->bytes = L->down_off + L->d_row * (size_t) n_embd;
    return MAYA_OK;
}

}  // extern "C"
