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

// Sequence numbers counted on the device (so that a captured CUDA graph can be replayed): a call made with seq == 0
// uses seq_counter[0] + 1, and the LAST block of the launch to finish stores it back - by then every block has read
// the counter.  seq_counter[1] is the launch's finishing ticket (zero between launches).
// The count skips 0 when it wraps (a zeroed word or flag would match it) by going from 0xffffffff to 2, which also keeps
// the two receive slots alternating (slot = seq & 1).
__device__ __forceinline__ unsigned ar_seq_next(unsigned c) { return c == 0xffffffffu ? 2u : c + 1u; }
__device__ __forceinline__ unsigned ar_seq_begin(const maya_peer_ar& a, unsigned seq) {
    return seq != 0u || a.seq_counter == nullptr ? seq : ar_seq_next(*(volatile unsigned*) a.seq_counter);
}
// every thread of the block calls this after the block's exchange
__device__ __forceinline__ void ar_seq_end(const maya_peer_ar& a, unsigned seq_arg, unsigned used) {
    if (seq_arg != 0u || a.seq_counter == nullptr) return;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&a.seq_counter[1], 1u) == gridDim.x - 1u) {
            a.seq_counter[1] = 0u;
            *(volatile unsigned*) a.seq_counter = used;
            __threadfence();
        }
    }
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
    // The block's stores reach the peers before the flags do: the barrier orders every thread's stores before the
    // flag-writing threads' system-scope fence (fences are cumulative), so only those few threads pay for one - a
    // system fence by all 1024 threads of all blocks cost the layer kernel several microseconds.
    __syncthreads();
    const size_t fslot = (size_t) slot * nm;
    if (tid < nm && tid != mi) {
        __threadfence_system();
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

// The same sum for SHORT vectors (the fused layer kernel: 40-odd floats a block), latency first: every float travels as
// one 64-bit store {seq, value} into the peers' word area (it follows the rows in the receive buffer: 2 x nm x stride
// 64-bit words, zeroed at start), and the receiver polls the word itself.  No fence, no separate flag: one NVLink
// one-way latency, where rows + flags cost a store round trip (the system fence) and then the flag's trip.  64-bit
// stores are single-copy atomic, the two slots alternate by seq as above (a word is overwritten two calls later, which
// the writer only reaches after this rank's reads of it); seq is never 0 (the device count skips it when it wraps,
// ar_seq_next; a host that counts must do the same).  Same bounded wait, error word and failure
// record.  Returns false when the transport is (or becomes) poisoned; x is then undefined.
__device__ __forceinline__ bool peer_allreduce_block_words(float* x, int q0, int q1, const maya_peer_ar& a, int mi,
                                                           unsigned seq, int b) {
    __shared__ int s_ready, s_failed;
    const int tid = threadIdx.x, nt = blockDim.x, nm = a.nm;
    if (tid == 0) { s_ready = (*(volatile unsigned*) a.error & 1u) == 0; s_failed = 0; }
    __syncthreads();
    if (!s_ready) return false;          // s_ready is not written again: every thread reads the same value
    const size_t slot = seq & 1u, words_off = (size_t) 2 * nm * a.stride;      // floats of row area before the words
    for (int t = tid; t < 4 * (q1 - q0); t += nt) {
        const size_t i = (size_t) 4 * q0 + t;
        const float mine = x[i];
        const unsigned long long word = ((unsigned long long) seq << 32) | __float_as_uint(mine);
        for (int m = 0; m < nm; ++m)
            if (m != mi)
                *((volatile unsigned long long*) (a.peer_recv[m] + words_off) + (slot * nm + mi) * a.stride + i) = word;
        const unsigned long long t0 = ar_global_ns();
        float acc = 0.0f;
        bool ok = true;
        for (int m = 0; m < nm && ok; ++m) {
            float p = mine;
            if (m != mi) {
                const volatile unsigned long long* src =
                    (const volatile unsigned long long*) (a.recv + words_off) + (slot * nm + m) * a.stride + i;
                unsigned long long w;
                while ((unsigned) ((w = *src) >> 32) != seq) {
                    const unsigned long long el = ar_global_ns() - t0;
                    if (el >= a.timeout_ns) {
                        if ((atomicOr(a.error, 1u) & 1u) == 0 && a.failure != nullptr) {
                            a.failure->sequence = seq;
                            a.failure->observed = (unsigned) (w >> 32);
                            a.failure->block = (unsigned) b;
                            a.failure->n4 = (unsigned) (q1 - q0);
                            a.failure->rank = (unsigned) mi;
                            a.failure->waited_for = (unsigned) m;
                            a.failure->elapsed_ns = el;
                            a.failure->timeout_ns = a.timeout_ns;
                            a.failure->captured = 1;
                        }
                        ok = false;
                        break;
                    }
                }
                p = __uint_as_float((unsigned) w);
            }
            acc = m == 0 ? p : __fadd_rn(acc, p);
        }
        if (ok) x[i] = acc;
        else s_failed = 1;
    }
    __syncthreads();
    return s_failed == 0;
}

}  // namespace maya
