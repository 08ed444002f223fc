// AVX-512-FP16 restatement of the reference's production attention kernel.  TEST
// INFRASTRUCTURE ONLY (timed CPU baseline and deviation report); never linked into
// the shipped library.  Compiled with -mavx512fp16 and guarded at run time.
//
//   oracle_f16_dot_product            src/kernel/x86_64/f16_512/dot_product.rs:7-19
//   oracle_f16_scalar_vector_mul_acc  src/kernel/x86_64/f16_512/flash_attention.rs:12-28
//   oracle_f16_flash_attention        src/kernel/x86_64/f16_512/flash_attention.rs:30-92
//   oracle_f16_attention_run_threads  item walk of src/compiler/mul/attention.rs:85-153
//                                     on the executor of src/serving/start.rs:37-73
//
// Everything - products, running max and sum, the divides, the output
// accumulators - is IEEE half, as in the reference; exp is float exp rounded to
// half (what Rust's f16::exp does).  head_size is fixed at 128 (four 32-lane
// accumulators), rows must be 64-byte aligned.

#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include <immintrin.h>
#include <pthread.h>
#include <sched.h>

#include "ellm_oracle.h"

namespace {

typedef _Float16 f16;

inline f16 f16_exp(f16 x) { return static_cast<f16>(std::exp(static_cast<float>(x))); }

inline f16 dot128(const f16* p1, const f16* p2, size_t length) {
    __m512h acc = _mm512_setzero_ph();
    for (size_t x = 0; x < length; x += 32) {
        __m512h x1 = _mm512_load_ph(p1 + x);
        __m512h x2 = _mm512_load_ph(p2 + x);
        acc = _mm512_fmadd_ph(x1, x2, acc);
    }
    return _mm512_reduce_add_ph(acc);
}

inline void axpy128(f16 scalar1, __m512h o[4], f16 scalar2, const f16* v) {
    __m512h s1 = _mm512_set1_ph(scalar1);
    __m512h s2 = _mm512_set1_ph(scalar2);
    for (int i = 0; i < 4; ++i) {
        __m512h vc = _mm512_load_ph(v + 32 * i);
        __m512h r2 = _mm512_mul_ph(s2, vc);
        o[i] = _mm512_fmadd_ph(s1, o[i], r2);
    }
}

inline void flash_row(const f16* q, const f16* K, const f16* V, f16* o, f16 inverse_sqrt_head,
                      size_t length, size_t stride, size_t position) {
    _mm_prefetch(reinterpret_cast<const char*>(K), _MM_HINT_T2);
    _mm_prefetch(reinterpret_cast<const char*>(K + 64), _MM_HINT_T2);
    _mm_prefetch(reinterpret_cast<const char*>(V), _MM_HINT_T2);
    _mm_prefetch(reinterpret_cast<const char*>(V + 64), _MM_HINT_T2);
    f16 m_i_1 = static_cast<f16>(-INFINITY);
    f16 d_i_1 = static_cast<f16>(0.0f);
    __m512h oc[4] = {_mm512_setzero_ph(), _mm512_setzero_ph(), _mm512_setzero_ph(),
                     _mm512_setzero_ph()};
    const size_t end = position * stride;
    for (size_t offset = 0; offset <= end; offset += stride) {
        if (offset < end) {
            const size_t next = offset + stride;
            _mm_prefetch(reinterpret_cast<const char*>(K + next), _MM_HINT_T2);
            _mm_prefetch(reinterpret_cast<const char*>(K + next + 64), _MM_HINT_T2);
            _mm_prefetch(reinterpret_cast<const char*>(V + next), _MM_HINT_T2);
            _mm_prefetch(reinterpret_cast<const char*>(V + next + 64), _MM_HINT_T2);
        }
        f16 x_i = dot128(q, K + offset, length);
        x_i = x_i * inverse_sqrt_head;
        f16 m_i = x_i > m_i_1 ? x_i : m_i_1;
        f16 update_exp = d_i_1 * f16_exp(m_i_1 - m_i);
        f16 add_exp = f16_exp(x_i - m_i);
        f16 d_i = update_exp + add_exp;
        f16 u = update_exp / d_i;
        f16 a = add_exp / d_i;
        axpy128(u, oc, a, V + offset);
        m_i_1 = m_i;
        d_i_1 = d_i;
    }
    for (int i = 0; i < 4; ++i) _mm512_store_ph(o + 32 * i, oc[i]);
}

struct SpinBarrier {
    alignas(64) std::atomic<size_t> arrived{0};
    alignas(64) std::atomic<size_t> generation{0};
    size_t tids;
    explicit SpinBarrier(size_t n) : tids(n) {}
    void wait() {
        size_t gen = generation.load(std::memory_order_relaxed);
        size_t a = arrived.fetch_add(1, std::memory_order_acq_rel) + 1;
        if (a == tids) {
            arrived.store(0, std::memory_order_relaxed);
            generation.store(gen + 1, std::memory_order_release);
            return;
        }
        while (generation.load(std::memory_order_acquire) == gen) __builtin_ia32_pause();
    }
};

void pin_to_core(size_t i) {
    cpu_set_t all;
    CPU_ZERO(&all);
    if (sched_getaffinity(0, sizeof(all), &all) != 0) return;
    int n = CPU_COUNT(&all);
    if (n <= 0) return;
    int want = static_cast<int>(i % static_cast<size_t>(n)), seen = 0;
    for (int c = 0; c < CPU_SETSIZE; ++c) {
        if (!CPU_ISSET(c, &all)) continue;
        if (seen++ == want) {
            cpu_set_t one;
            CPU_ZERO(&one);
            CPU_SET(c, &one);
            pthread_setaffinity_np(pthread_self(), sizeof(one), &one);
            return;
        }
    }
}

}  // namespace

extern "C" {

int oracle_f16_available(void) { return __builtin_cpu_supports("avx512fp16") ? 1 : 0; }

float oracle_f16_dot_product(const uint16_t* a, const uint16_t* b, size_t length) {
    if (!oracle_f16_available()) return 0.0f;
    return static_cast<float>(
        dot128(reinterpret_cast<const f16*>(a), reinterpret_cast<const f16*>(b), length));
}

void oracle_f16_scalar_vector_mul_acc(float scalar1, uint16_t* o128, float scalar2,
                                      const uint16_t* v128) {
    if (!oracle_f16_available()) return;
    f16* o = reinterpret_cast<f16*>(o128);
    __m512h oc[4];
    for (int i = 0; i < 4; ++i) oc[i] = _mm512_load_ph(o + 32 * i);
    axpy128(static_cast<f16>(scalar1), oc, static_cast<f16>(scalar2),
            reinterpret_cast<const f16*>(v128));
    for (int i = 0; i < 4; ++i) _mm512_store_ph(o + 32 * i, oc[i]);
}

void oracle_f16_flash_attention(const uint16_t* q, const uint16_t* K, const uint16_t* V,
                                uint16_t* o, float inverse_sqrt_head, size_t length,
                                size_t stride, size_t position) {
    if (!oracle_f16_available()) return;
    flash_row(reinterpret_cast<const f16*>(q), reinterpret_cast<const f16*>(K),
              reinterpret_cast<const f16*>(V), reinterpret_cast<f16*>(o),
              static_cast<f16>(inverse_sqrt_head), length, stride, position);
}

double oracle_f16_attention_run_threads(const uint16_t* q, const uint16_t* k, const uint16_t* v,
                                        uint16_t* out, const int32_t* positions,
                                        size_t max_batch, size_t q_heads, size_t kv_heads,
                                        const size_t* kv_strides, float scale,
                                        size_t position_index, size_t position_interval,
                                        size_t batch_size, size_t threads, size_t repeats) {
    if (!oracle_f16_available()) return -1.0;
    if (threads == 0) threads = std::thread::hardware_concurrency();
    if (threads == 0) threads = 1;
    if (repeats == 0) repeats = 1;
    const size_t D = 128, group = q_heads / kv_heads;
    const size_t s0 = kv_strides[0], s1 = kv_strides[1], s2 = kv_strides[2];
    SpinBarrier barrier(threads);
    std::vector<std::thread> pool;
    std::chrono::steady_clock::time_point t0, t1;
    for (size_t t = 0; t < threads; ++t) {
        pool.emplace_back([&, t]() {
            pin_to_core(t);
            barrier.wait();
            if (t == 0) t0 = std::chrono::steady_clock::now();
            for (size_t rep = 0; rep < repeats; ++rep) {
                const size_t stride = batch_size * q_heads;
                size_t begin, end;
                if (oracle_assign(position_interval * stride, threads, t, &begin, &end)) {
                    const size_t max_stride = max_batch * q_heads;
                    size_t high = begin / stride, rem = begin % stride;
                    size_t row = rem / q_heads, col = rem % q_heads;
                    for (size_t it = begin; it < end; ++it) {
                        const size_t index = (high * max_stride + row * q_heads + col) * D;
                        const size_t kv_index = row * s0 + (col / group) * s1;
                        const size_t base =
                            positions ? static_cast<size_t>(positions[row]) : position_index;
                        flash_row(reinterpret_cast<const f16*>(q) + index,
                                  reinterpret_cast<const f16*>(k) + kv_index,
                                  reinterpret_cast<const f16*>(v) + kv_index,
                                  reinterpret_cast<f16*>(out) + index, static_cast<f16>(scale), D,
                                  s2, base + high);
                        if (++col == q_heads) { col = 0; ++row; }
                        if (row == batch_size) { row = 0; ++high; }
                    }
                }
                barrier.wait();  // the executor's per-operator barrier
            }
            if (t == 0) t1 = std::chrono::steady_clock::now();
        });
    }
    for (auto& th : pool) th.join();
    return std::chrono::duration<double>(t1 - t0).count();
}

}  // extern "C"
