// allreduce.cu - the cross-GPU sum of expert partials over NVLink peer memory: every rank stores its vector into a
// receive slot in EVERY peer's own HBM, raises a flag there, waits (bounded) for the peers' flags in its own memory
// and adds the nm vectors in rank order, so all ranks end with the same bits.
//
// Generalises the reference's two-rank peer push/reduce (ar_peer_kernel, src/ds4/ds4_kernels.cu:3530-3585; PeerAr,
// src/ds4/ds4_kernels.cuh:523-547) to nm <= 8 ranks and keeps its contract: two receive slots used alternately by
// `seq & 1`; one call per rank per seq on one stream, same n everywhere, no skipped calls; flags start at
// first_seq - 1; a wait that outlasts `timeout_ns` sets the sticky error word (and fills the optional failure
// record) and every later call on that transport returns at once; the sum is member 0 + member 1 + ... with
// round-to-nearest adds (ar_sum_kernel's order, ds4_kernels.cu:3503-3526).
//
// Only plain stores to peer-mapped addresses and plain loads of local memory are used: no TMA, no multicast, no
// loads from a peer's memory.
#include <cstring>

#include "maya_internal.cuh"
#include "maya_peer_ar.cuh"

namespace maya {
namespace {

__global__ void __launch_bounds__(256) ar_peer_kernel(float* x, int n4, maya_peer_ar a, int mi, unsigned seq) {
    const int nb = gridDim.x, b = blockIdx.x;
    const int base = n4 / nb, rem = n4 % nb;
    const int q0 = b * base + min(b, rem), q1 = q0 + base + (b < rem ? 1 : 0);
    peer_allreduce_block(x, q0, q1, a, mi, seq, b);
}

// touches nothing: loads the kernel image so that no rank meets CUDA's lazy loading while another already spins
__global__ void ar_preload_kernel() {}

}  // namespace
}  // namespace maya

using namespace maya;

extern "C" size_t maya_peer_ar_recv_bytes(int nm, size_t stride) {
    if (nm < 1 || nm > MAYA_PEER_AR_MAX_RANKS || stride == 0) return 0;
    // two slots of nm rows, then the same again as 64-bit {seq, value} words (the fused layer kernel's exchange)
    return (size_t) 2 * nm * stride * (sizeof(float) + sizeof(unsigned long long));
}
extern "C" size_t maya_peer_ar_flag_bytes(int nm) {
    if (nm < 1 || nm > MAYA_PEER_AR_MAX_RANKS) return 0;
    return (size_t) 2 * nm * MAYA_PEER_AR_BLOCKS * MAYA_PEER_AR_FLAG_STRIDE * sizeof(unsigned);
}

extern "C" int maya_peer_ar_preload(void* stream) {
    ar_preload_kernel<<<1, 32, 0, as_stream(stream)>>>();
    int st = note_launch("peer_ar_preload");
    if (st != MAYA_OK) return st;
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, ar_peer_kernel) != cudaSuccess) return note_launch("peer_ar_preload attributes");
    return MAYA_OK;
}

extern "C" int maya_allreduce_peer(float* x, int n, const maya_peer_ar* a, int mi, unsigned seq, void* stream) {
    if (!x || !a || !a->recv || !a->peer_recv || !a->flags || !a->peer_flags || !a->error) return refuse(MAYA_ERR_ARG);
    if (a->nm < 2 || a->nm > MAYA_PEER_AR_MAX_RANKS || mi < 0 || mi >= a->nm) return refuse(MAYA_ERR_ARG);
    if (n <= 0 || n % 4 || (size_t) n > a->stride || !aligned16(x) || a->stride % 4) return refuse(MAYA_ERR_ARG);
    if (a->timeout_ns == 0) return refuse(MAYA_ERR_ARG);
    const int n4 = n / 4;
    int blocks = (n4 + 255) / 256;
    if (blocks > 64) blocks = 64;
    ar_peer_kernel<<<blocks, 256, 0, as_stream(stream)>>>(x, n4, *a, mi, seq);
    return note_launch("allreduce_peer");
}

// ---------------------------------------------------------------- set-up helpers (not on the token path)
extern "C" int maya_peer_buffer_create(size_t bytes, void** ptr, unsigned char handle[64]) {
    if (!ptr || !handle || bytes == 0) return MAYA_ERR_ARG;
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return note_launch("peer_buffer_create malloc");
    if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {   // flags start at 0
        cudaFree(p);
        return note_launch("peer_buffer_create memset");
    }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaFree(p); return note_launch("peer_buffer_create handle"); }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    std::memcpy(handle, &h, 64);
    *ptr = p;
    return MAYA_OK;
}
extern "C" int maya_peer_buffer_open(const unsigned char handle[64], void** ptr) {
    if (!ptr || !handle) return MAYA_ERR_ARG;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    if (cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return note_launch("peer_buffer_open");
    return MAYA_OK;
}
extern "C" int maya_peer_buffer_close(void* ptr) {
    if (ptr && cudaIpcCloseMemHandle(ptr) != cudaSuccess) return note_launch("peer_buffer_close");
    return MAYA_OK;
}
extern "C" int maya_peer_buffer_destroy(void* ptr) {
    if (ptr && cudaFree(ptr) != cudaSuccess) return note_launch("peer_buffer_destroy");
    return MAYA_OK;
}
