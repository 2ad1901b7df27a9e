// ref_shim_layer.cpp - TEST INFRASTRUCTURE (bench.py's CPU arm; nothing the library ships uses it).
//
// One decode token of a MoE layer on the host cores, the way the reference's CPU expert lane computes it: the routed
// experts through the reference's OWN AVX-512 / AVX2 rows (src/kernels/cpu/iq_avx512.cpp, iq_avx2.cpp: iq512_gu_rows,
// iq512_rows) over Q8_K activations (its host transcription of ggml's quantizer, ref_shim_q8k.cpp), every expert's rows
// split across all threads as its pool does (include/strata/kernels/cpu/pool.hpp:120,
// include/strata/core/expert_source.hpp:218), on a persistent thread pool; the weighted sum in plan order.
//
// The reference hands Q8_0 weights (the shared expert of the headline configuration) to ggml-cpu, whose source is not
// in its tree.  The shared expert therefore runs through the AVX2 dot below: q8_1 activations (d = amax / 127, the CUDA
// path's quantizer), per 32-value block an exact int8 dot (sign / maddubs / madd) scaled by the two f16 scales - the
// arithmetic of the reference's CUDA Q8_0 dot (src/kernels/cuda/native_mmvq.cu:708-720) on the host.
#include <immintrin.h>

#include <atomic>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#include "strata/kernels/cpu/iq_avx2.hpp"
#include "strata/kernels/cpu/iq_avx512.hpp"

#define REF_API extern "C" __attribute__((visibility("default")))
using namespace strata::kernels::cpu;

extern "C" void ref_quantize_q8_K(const float* x, long long n, unsigned char* blocks);

namespace {

// ---------------------------------------------------------------- a persistent pool: run(n, f) calls f(0..n-1)
class Pool {
public:
    explicit Pool(int n) : n_(n < 1 ? 1 : n) {
        for (int i = 1; i < n_; ++i) workers_.emplace_back([this] { loop(); });
    }
    ~Pool() {
        {
            std::lock_guard<std::mutex> g(m_);
            stop_ = true;
            ++gen_;
        }
        cv_.notify_all();
        for (auto& t : workers_) t.join();
    }
    int size() const { return n_; }
    void run(int chunks, const std::function<void(int)>& f) {
        {
            std::lock_guard<std::mutex> g(m_);
            f_ = &f;
            chunks_ = chunks;
            next_.store(0);
            left_.store(n_ - 1);
            ++gen_;
        }
        cv_.notify_all();
        work();
        while (left_.load(std::memory_order_acquire) != 0) _mm_pause();
    }

private:
    void work() {
        for (;;) {
            const int c = next_.fetch_add(1);
            if (c >= chunks_) break;
            (*f_)(c);
        }
    }
    void loop() {
        unsigned long long seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> g(m_);
                cv_.wait(g, [&] { return gen_ != seen; });
                seen = gen_;
                if (stop_) return;
            }
            work();
            left_.fetch_sub(1, std::memory_order_release);
        }
    }
    int n_;
    std::vector<std::thread> workers_;
    std::mutex m_;
    std::condition_variable cv_;
    unsigned long long gen_ = 0;
    bool stop_ = false;
    const std::function<void(int)>* f_ = nullptr;
    int chunks_ = 0;
    std::atomic<int> next_{0}, left_{0};
};

// ---------------------------------------------------------------- Q8_0 weights x q8_1 activations, AVX2
struct Q81 { float d; int8_t q[32]; };   // host form of a q8_1 block: the f16-rounded scale kept as f32

void quantize_q8_1(const float* x, int n, Q81* y) {
    for (int b = 0; b < n / 32; ++b) {
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) amax = std::fmax(amax, std::fabs(x[b * 32 + i]));
        const float d = std::fmin(amax / 127.0f, 65504.0f);
        for (int i = 0; i < 32; ++i) {
            const float v = amax == 0.0f ? 0.0f : std::round(x[b * 32 + i] / d);
            y[b].q[i] = (int8_t) std::fmax(-127.0f, std::fmin(127.0f, v));
        }
        y[b].d = _cvtsh_ss(_cvtss_sh(d, _MM_FROUND_TO_NEAREST_INT));
    }
}

float dot_q8_0(const uint8_t* row, const Q81* x, int nblk) {
    __m256 acc = _mm256_setzero_ps();
    for (int b = 0; b < nblk; ++b) {
        const uint8_t* blk = row + (size_t) b * 34;
        uint16_t dh;
        std::memcpy(&dh, blk, 2);
        const __m256i w = _mm256_loadu_si256((const __m256i*) (blk + 2));
        const __m256i a = _mm256_loadu_si256((const __m256i*) x[b].q);
        const __m256i aw = _mm256_sign_epi8(w, w);                 // |w|
        const __m256i sa = _mm256_sign_epi8(a, w);                 // a * sign(w)
        const __m256i p16 = _mm256_maddubs_epi16(aw, sa);
        const __m256i p32 = _mm256_madd_epi16(p16, _mm256_set1_epi16(1));
        const float d = _cvtsh_ss(dh) * x[b].d;
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(p32), acc);
    }
    __m128 s = _mm_add_ps(_mm256_castps256_ps128(acc), _mm256_extractf128_ps(acc, 1));
    s = _mm_add_ps(s, _mm_movehl_ps(s, s));
    s = _mm_add_ss(s, _mm_movehdup_ps(s));
    return _mm_cvtss_f32(s);
}

float silu_mul(float g, float u) { return g / (1.0f + std::exp(-g)) * u; }

void gu_rows(int avx512, int t, const uint8_t* blob, size_t gu_row, size_t up_off, int n, const void* a, float* ff, int r0, int r1) {
    const void* acts[1] = {a};
    float* outs[1] = {ff};
    if (avx512) iq512_gu_rows(t, blob, gu_row, up_off, n, acts, 1, outs, r0, r1);
    else iq256_gu_rows(t, blob, gu_row, up_off, n, acts, 1, outs, r0, r1);
}
void rows(int avx512, int t, const uint8_t* w, size_t rb, int n, const void* a, float* out, int r0, int r1) {
    const void* acts[1] = {a};
    float* outs[1] = {out};
    if (avx512) iq512_rows(t, w, rb, n, acts, 1, outs, r0, r1);
    else iq256_rows(t, w, rb, n, acts, 1, outs, r0, r1);
}

Pool* g_pool = nullptr;

}  // namespace

REF_API int ref_pool_threads(int threads) {
    if (g_pool == nullptr || g_pool->size() != threads) {
        delete g_pool;
        g_pool = new Pool(threads);
    }
    return g_pool->size();
}

// n_tok tokens, one after another.  blobs[t * k + j]: token t's j-th routed expert ([gate | up | down] rows of
// gu_type / d_type); w[t * k + j] its weight; x[t * n_embd ..]; shared: the Q8_0 shared expert's blob or NULL.
// out[t * n_embd ..].  Returns the seconds the n_tok tokens took (quantizing, experts, combine).
REF_API double ref_layer_tokens(int avx512, int gu_type, int d_type, size_t gu_row, size_t d_row, int n_embd, int n_ff, int k,
                                const uint8_t* const* blobs, const float* w, const float* x, const uint8_t* shared, int n_ff_sh,
                                int n_tok, float* out) {
    if (g_pool == nullptr) ref_pool_threads((int) std::thread::hardware_concurrency());
    Pool& P = *g_pool;
    const int nth = P.size();
    std::vector<uint8_t> a((size_t) n_embd / 256 * 292), hq((size_t) k * (n_ff / 256) * 292);
    std::vector<float> h((size_t) k * n_ff), part((size_t) k * n_embd), sh_h(n_ff_sh > 0 ? n_ff_sh : 1), sh_out(n_embd);
    std::vector<Q81> xq1(n_embd / 32), shq1(n_ff_sh > 0 ? n_ff_sh / 32 : 1);
    const size_t sh_rb = (size_t) n_embd / 32 * 34, sh_drb = (size_t) (n_ff_sh > 0 ? n_ff_sh : 32) / 32 * 34;
    auto split = [&](int n, int c, int& r0, int& r1) {
        const int step = (n + nth - 1) / nth;
        r0 = c * step < n ? c * step : n;
        r1 = r0 + step < n ? r0 + step : n;
    };
    const auto t0 = std::chrono::steady_clock::now();
    for (int t = 0; t < n_tok; ++t) {
        const float* xt = x + (size_t) t * n_embd;
        ref_quantize_q8_K(xt, n_embd, a.data());
        if (shared) quantize_q8_1(xt, n_embd, xq1.data());
        // gate/up + SwiGLU: every expert's FFN rows split over all threads; the shared expert's rows likewise
        P.run((k + (shared ? 1 : 0)) * nth, [&](int c) {
            const int j = c / nth;
            int r0, r1;
            if (j < k) {
                split(n_ff, c % nth, r0, r1);
                if (r0 < r1) gu_rows(avx512, gu_type, blobs[t * k + j], gu_row, (size_t) n_ff * gu_row, n_embd, a.data(), h.data() + (size_t) j * n_ff, r0, r1);
            } else {
                split(n_ff_sh, c % nth, r0, r1);
                for (int r = r0; r < r1; ++r)
                    sh_h[r] = silu_mul(dot_q8_0(shared + (size_t) r * sh_rb, xq1.data(), n_embd / 32),
                                       dot_q8_0(shared + (size_t) (n_ff_sh + r) * sh_rb, xq1.data(), n_embd / 32));
            }
        });
        for (int j = 0; j < k; ++j) ref_quantize_q8_K(h.data() + (size_t) j * n_ff, n_ff, hq.data() + (size_t) j * (n_ff / 256) * 292);
        if (shared) quantize_q8_1(sh_h.data(), n_ff_sh, shq1.data());
        P.run((k + (shared ? 1 : 0)) * nth, [&](int c) {
            const int j = c / nth;
            int r0, r1;
            split(n_embd, c % nth, r0, r1);
            if (j < k) {
                if (r0 < r1) rows(avx512, d_type, blobs[t * k + j] + 2 * (size_t) n_ff * gu_row, d_row, n_ff, hq.data() + (size_t) j * (n_ff / 256) * 292,
                                  part.data() + (size_t) j * n_embd, r0, r1);
            } else {
                const uint8_t* down = shared + 2 * (size_t) n_ff_sh * sh_rb;
                for (int r = r0; r < r1; ++r) sh_out[r] = dot_q8_0(down + (size_t) r * sh_drb, shq1.data(), n_ff_sh / 32);
            }
        });
        float* o = out + (size_t) t * n_embd;
        for (int r = 0; r < n_embd; ++r) {
            float m = 0.0f;
            for (int j = 0; j < k; ++j) m += w[t * k + j] * part[(size_t) j * n_embd + r];
            o[r] = m + (shared ? sh_out[r] : 0.0f);
        }
    }
    return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
}
