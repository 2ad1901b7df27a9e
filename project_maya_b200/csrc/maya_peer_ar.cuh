// maya_peer_ar.cuh - the device side of the peer-memory all-reduce, shared by the stand-alone kernel (allreduce.cu)
// and the fused layer kernel's epilogue (moe_fused.cu).  See allreduce.cu for the protocol and its contract.
#pragma once

#include "maya_common.cuh"

namespace maya {

__device__ __forceinline__ unsigned long long ar_global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ float4 ld_fresh4(const float4* p) {   // bypass L1: the bytes came from another GPU
    float4 v;
    asm volatile("ld.global.cv.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

// Device-side protocol for one block's share [q0, q1) (in float4 units) of the vector; block index `b` picks the flag
// word.  Callable from the stand-alone kernel and from the fused layer kernel's epilogue.  Returns false when the
// transport is (or becomes) poisoned; x is then left as the local partial.
__device__ __forceinline__ bool peer_allreduce_block(float* x, int q0, int q1, const maya_peer_ar& a, int mi, unsigned seq, int b) {
    __shared__ int s_ready;
    const int tid = threadIdx.x, nt = blockDim.x, nm = a.nm;
    if (tid == 0) s_ready = (*(volatile unsigned*) a.error & 1u) == 0;
    __syncthreads();
    if (!s_ready) return false;
    const int slot = (int) (seq & 1u);
    const size_t row = ((size_t) slot * nm + mi) * a.stride;           // my row inside a peer's receive buffer
    for (int m = 0; m < nm; ++m) {
        if (m == mi) continue;
        float4* dst = (float4*) (a.peer_recv[m] + row);
        for (int q = q0 + tid; q < q1; q += nt) dst[q] = ((const float4*) x)[q];
    }
    __threadfence_system();          // my stores reach the peers before the flags do
    __syncthreads();
    const size_t fslot = (size_t) slot * nm;
    if (tid < nm && tid != mi) {
        volatile unsigned* f = a.peer_flags[tid] + ((fslot + mi) * MAYA_PEER_AR_BLOCKS + b) * MAYA_PEER_AR_FLAG_STRIDE;
        *f = seq;
    }
    if (tid < nm && tid != mi) {
        const volatile unsigned* f = a.flags + ((fslot + tid) * MAYA_PEER_AR_BLOCKS + b) * MAYA_PEER_AR_FLAG_STRIDE;
        const unsigned long long t0 = ar_global_ns();
        unsigned seen;
        while ((int) ((seen = *f) - seq) < 0) {
            const unsigned long long el = ar_global_ns() - t0;
            if (el >= a.timeout_ns) {
                if ((atomicOr(a.error, 1u) & 1u) == 0 && a.failure != nullptr) {
                    a.failure->sequence = seq;
                    a.failure->observed = seen;
                    a.failure->block = (unsigned) b;
                    a.failure->n4 = (unsigned) (q1 - q0);
                    a.failure->rank = (unsigned) mi;
                    a.failure->waited_for = (unsigned) tid;
                    a.failure->elapsed_ns = el;
                    a.failure->timeout_ns = a.timeout_ns;
                    a.failure->captured = 1;
                }
                s_ready = 0;
                break;
            }
        }
        __threadfence_system();
    }
    __syncthreads();
    if (!s_ready) return false;
    for (int q = q0 + tid; q < q1; q += nt) {
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int m = 0; m < nm; ++m) {
            const float4 p = m == mi ? ((const float4*) x)[q]
                                     : ld_fresh4((const float4*) (a.recv + ((size_t) slot * nm + m) * a.stride) + q);
            if (m == 0) v = p;
            else { v.x = __fadd_rn(v.x, p.x); v.y = __fadd_rn(v.y, p.y); v.z = __fadd_rn(v.z, p.z); v.w = __fadd_rn(v.w, p.w); }
        }
        ((float4*) x)[q] = v;
    }
    return true;
}


}  // namespace maya
