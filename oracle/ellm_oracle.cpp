// CPU oracle for the eLLM attention path.  TEST INFRASTRUCTURE ONLY: this file
// is the checker the CUDA path is compared against and the CPU baseline that
// the benchmark times; nothing in the shipped library links or calls it.
//
// Every function restates, in plain C++, one function of the reference crate
// (paths are relative to the reference project root):
//
//   oracle_dot_product_f32        src/kernel/generic/flash_attention.rs:17-28
//   oracle_scalar_vector_mul_acc  src/kernel/generic/flash_attention.rs:39-47
//   oracle_flash_attention_f32    src/kernel/generic/flash_attention.rs:60-89
//   oracle_assign                 src/compiler/assign.rs:11-38
//   oracle_attention_run_*        src/compiler/mul/attention.rs:69-156 (the
//                                 commented-out body of Attention::run) driven
//                                 like src/serving/start.rs:37-73 with the spin
//                                 barrier of src/runtime/barrier.rs:25-40
//   oracle_kv_append              row write at [position] with the semantics of
//                                 the output_to_kv branch,
//                                 src/compiler/zip_map/complex_zip.rs:92-98
//   oracle_rms_norm_f32           src/kernel/generic/rms_norm.rs:6-26
//   oracle_complex_mul_f32        src/kernel/generic/complex_mul.rs:3-20
//   oracle_precompute_freqs_cis   src/qwen3_moe/rope.rs:7-28
//   oracle_qk_norm_rope_append    src/kernel/x86_64/f16_512/matmul_rms_complex.rs:76-96
//   oracle_matmul_nt_bf16         src/compiler/mul/matmul_add.rs:128-232 (C = residual, C += A x B),
//                                 src/compiler/mul/matmul3.rs:289-385 (the three projections)
//
// Pinning.  The reference's own tests for this path hold only uniform-input
// known-answer cases (all-ones attention -> all-ones output, 1*1+2*2=5,
// [1,2,3].[4,5,6]=32, the assign() splits).  The oracle reproduces all of them
// (tests/test_oracle_kat.py).  They do not pin the softmax scale, the causal
// limit, the grouped-query head mapping or the LSE, so for non-uniform inputs
// the oracle is additionally cross-checked against an independent float64
// two-pass softmax.  The reference itself (Rust nightly) cannot be compiled
// where this builds.
//
// Three deliberate departures from the reference text, each switchable or
// documented here so the difference is visible:
//   1. generic/flash_attention.rs:76 exponentiates the UNSCALED score while the
//      running maximum (line 72-73) uses the scaled one.  With `faithful_scale_
//      defect == 0` (the default, and what parity uses) both use the scaled
//      score, as the AVX-512-FP16 kernel of the same crate does
//      (x86_64/f16_512/flash_attention.rs:70-77).  Non-zero reproduces line 76.
//   2. attention.rs:129 maps a query head to `col / kv_head_num`; grouped-query
//      attention needs `col / (q_heads / kv_heads)`.  The oracle uses the latter.
//   3. attention.rs:96-103 offsets K/V by `position_index * kv_strides[position_
//      index]`; a query row at absolute position p must see keys 0..=p, so the
//      base offset is 0 here.
// The running (m, d) of the recurrence are returned as LSE = m + ln(d); the
// reference drops them.

#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include <pthread.h>
#include <sched.h>

#include "ellm_oracle.h"

namespace {

inline float bf16_to_f32(uint16_t h) {
    uint32_t u = static_cast<uint32_t>(h) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

// round-to-nearest-even, NaN kept quiet
inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return static_cast<uint16_t>(u >> 16);
}

// src/runtime/barrier.rs:7-40: arrival counter + generation word, spin on the
// generation.
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
        while (generation.load(std::memory_order_acquire) == gen) {
#if defined(__x86_64__)
            __builtin_ia32_pause();
#endif
        }
    }
};

void pin_to_core(size_t i) {
    cpu_set_t all;
    CPU_ZERO(&all);
    if (sched_getaffinity(0, sizeof(all), &all) != 0) return;
    int n = CPU_COUNT(&all);
    if (n <= 0) return;
    int want = static_cast<int>(i % static_cast<size_t>(n));
    int seen = 0;
    for (int c = 0; c < CPU_SETSIZE; ++c) {
        if (!CPU_ISSET(c, &all)) continue;
        if (seen == want) {
            cpu_set_t one;
            CPU_ZERO(&one);
            CPU_SET(c, &one);
            pthread_setaffinity_np(pthread_self(), sizeof(one), &one);
            return;
        }
        ++seen;
    }
}

}  // namespace

extern "C" {

float oracle_dot_product_f32(const float* a, const float* b, size_t length) {
    float result = 0.0f;
    for (size_t i = 0; i < length; ++i) result = result + a[i] * b[i];
    return result;
}

void oracle_scalar_vector_mul_acc_f32(float scalar1, float* o, float scalar2, const float* v,
                                      size_t length) {
    for (size_t i = 0; i < length; ++i) o[i] = scalar1 * o[i] + scalar2 * v[i];
}

void oracle_flash_attention_f32(const float* q, const float* K, const float* V, float* o,
                                float inverse_sqrt_head, size_t length, size_t stride,
                                size_t position, int faithful_scale_defect, float* lse_out) {
    float m_i_1 = -INFINITY;
    float d_i_1 = 0.0f;
    size_t offset = 0;
    for (size_t i = 0; i <= position; ++i) {
        float x_i = oracle_dot_product_f32(q, K + offset, length);
        float scale_x_i = x_i * inverse_sqrt_head;
        float m_i = scale_x_i > m_i_1 ? scale_x_i : m_i_1;
        float update_exp = d_i_1 * std::exp(m_i_1 - m_i);
        float add_exp = std::exp((faithful_scale_defect ? x_i : scale_x_i) - m_i);
        float d_i = update_exp + add_exp;
        float u = update_exp / d_i;
        float a = add_exp / d_i;
        oracle_scalar_vector_mul_acc_f32(u, o, a, V + offset, length);
        m_i_1 = m_i;
        d_i_1 = d_i;
        offset += stride;
    }
    if (lse_out) *lse_out = m_i_1 + std::log(d_i_1);
}

int oracle_assign(size_t length, size_t num, size_t id, size_t* begin, size_t* end) {
    if (num == 0 || id >= num) return 0;
    if (length < id + 1) return 0;
    size_t quotient = length / num, remainder = length % num;
    if (remainder == 0) {
        *begin = quotient * id;
        *end = *begin + quotient;
        return 1;
    }
    if (id < remainder) {
        *begin = (quotient + 1) * id;
        *end = *begin + quotient + 1;
        return 1;
    }
    *begin = quotient * id + remainder;
    *end = *begin + quotient;
    return 1;
}

// One thread's share of Attention::run (attention.rs:85-153): flat items
// (high_index = row of the chunk, row_index = sequence in the batch, col_index =
// query head), head fastest; q/out are addressed with the MAX batch stride, K/V
// with kv_strides[0] per sequence and kv_strides[1] per KV head; the causal
// limit of an item is position_index + high_index; when per-sequence positions
// are given (the C ABI's ragged extension) positions[row] replaces position_index.
void oracle_attention_run_bf16(const oracle_attn_desc* d, size_t position_index,
                               size_t position_interval, size_t batch_size, size_t cpu_num,
                               size_t thread_id) {
    const size_t Hq = d->q_heads, Hkv = d->kv_heads, D = d->head_size;
    const size_t group = Hq / Hkv;
    const size_t stride = batch_size * Hq;
    size_t begin, end;
    if (!oracle_assign(position_interval * stride, cpu_num, thread_id, &begin, &end)) return;
    const size_t max_stride = d->max_batch * Hq;
    size_t high_index = begin / stride, rem = begin % stride;
    size_t row_index = rem / Hq, col_index = rem % Hq;

    std::vector<float> qf(D), of(D);
    std::vector<float> kf, vf;
    size_t cached_row = SIZE_MAX, cached_kvh = SIZE_MAX, cached_n = 0;

    for (size_t it = begin; it < end; ++it) {
        const size_t index = (high_index * max_stride + row_index * Hq + col_index) * D;
        const size_t kvh = col_index / group;
        const size_t kv_index = row_index * d->kv_strides[0] + kvh * d->kv_strides[1];
        const size_t base =
            d->positions ? static_cast<size_t>(d->positions[row_index]) : position_index;
        const size_t position = base + high_index;
        // widen the K/V rows this item reads once per (sequence, kv head)
        const size_t n = position + 1;
        if (cached_row != row_index || cached_kvh != kvh || cached_n < n) {
            const size_t want = base + position_interval;  // most rows any item of the chunk reads
            kf.resize(want * D);
            vf.resize(want * D);
            for (size_t r = 0; r < want; ++r) {
                const uint16_t* kr = d->k + kv_index + r * d->kv_strides[2];
                const uint16_t* vr = d->v + kv_index + r * d->kv_strides[2];
                for (size_t c = 0; c < D; ++c) {
                    kf[r * D + c] = bf16_to_f32(kr[c * d->kv_strides[3]]);
                    vf[r * D + c] = bf16_to_f32(vr[c * d->kv_strides[3]]);
                }
            }
            cached_row = row_index;
            cached_kvh = kvh;
            cached_n = want;
        }
        for (size_t c = 0; c < D; ++c) {
            qf[c] = bf16_to_f32(d->q[index + c]);
            of[c] = 0.0f;
        }
        float lse = 0.0f;
        oracle_flash_attention_f32(qf.data(), kf.data(), vf.data(), of.data(), d->scale, D, D,
                                   position, 0, &lse);
        for (size_t c = 0; c < D; ++c) d->out[index + c] = f32_to_bf16(of[c]);
        if (d->lse) d->lse[index / D] = lse;

        if (++col_index == Hq) {
            col_index = 0;
            ++row_index;
        }
        if (row_index == batch_size) {
            row_index = 0;
            ++high_index;
        }
    }
}

// The executor of src/serving/start.rs:37-73 for one operator: `threads` pinned
// threads each call run(position_index, position_interval, batch, threads, tid)
// and meet at the spin barrier.
void oracle_attention_run_threads_bf16(const oracle_attn_desc* d, size_t position_index,
                                       size_t position_interval, size_t batch_size,
                                       size_t threads) {
    if (threads == 0) threads = std::thread::hardware_concurrency();
    if (threads == 0) threads = 1;
    SpinBarrier barrier(threads);
    std::vector<std::thread> pool;
    pool.reserve(threads);
    for (size_t t = 0; t < threads; ++t) {
        pool.emplace_back([=, &barrier]() {
            pin_to_core(t);
            oracle_attention_run_bf16(d, position_index, position_interval, batch_size, threads, t);
            barrier.wait();
        });
    }
    for (auto& th : pool) th.join();
}

// Row write of the chunk's new K (or V) rows into the static cache:
// src[(h*max_batch + b)*Hkv + kvh][D] -> cache[b*s0 + kvh*s1 + (pos_b + h)*s2 + c*s3]
// with pos_b = position_index, or positions[b] when ragged.
void oracle_kv_append_bf16(uint16_t* cache, const uint16_t* src, const size_t* kv_strides,
                           size_t max_batch, size_t kv_heads, size_t head_size,
                           size_t position_index, size_t position_interval, size_t batch_size,
                           const int32_t* positions) {
    for (size_t h = 0; h < position_interval; ++h)
        for (size_t b = 0; b < batch_size; ++b) {
            size_t pos = (positions ? static_cast<size_t>(positions[b]) : position_index) + h;
            for (size_t kvh = 0; kvh < kv_heads; ++kvh) {
                const uint16_t* s = src + ((h * max_batch + b) * kv_heads + kvh) * head_size;
                uint16_t* dst = cache + b * kv_strides[0] + kvh * kv_strides[1] + pos * kv_strides[2];
                for (size_t c = 0; c < head_size; ++c) dst[c * kv_strides[3]] = s[c];
            }
        }
}

// (O, LSE) partial combine, the exchange step of the sequence-chunk sharding.
// No counterpart in the reference (it has no split); stated here so the GPU
// merge kernel has a CPU checker:  L = log(sum_i exp(L_i)),  O = sum_i O_i exp(L_i - L).
void oracle_merge_partials_f32(const float* o_parts, const float* lse_parts, size_t parts,
                               size_t rows, size_t head_size, float* o, float* lse) {
    for (size_t r = 0; r < rows; ++r) {
        float m = -INFINITY;
        for (size_t p = 0; p < parts; ++p) m = std::fmax(m, lse_parts[p * rows + r]);
        double s = 0.0;
        for (size_t p = 0; p < parts; ++p) {
            float l = lse_parts[p * rows + r];
            if (l != -INFINITY) s += std::exp(static_cast<double>(l) - m);
        }
        float L = (m == -INFINITY) ? -INFINITY : m + static_cast<float>(std::log(s));
        for (size_t c = 0; c < head_size; ++c) {
            double acc = 0.0;
            for (size_t p = 0; p < parts; ++p) {
                float l = lse_parts[p * rows + r];
                if (l == -INFINITY) continue;
                acc += static_cast<double>(o_parts[(p * rows + r) * head_size + c]) *
                       std::exp(static_cast<double>(l) - L);
            }
            o[r * head_size + c] = static_cast<float>(acc);
        }
        lse[r] = L;
    }
}

// ---- the step before attention: per-head RMSNorm + interleaved RoPE + cache write ----

// src/kernel/generic/rms_norm.rs:6-26: y = x / (sqrt(mean(x^2)) + eps) - note eps is added to
// the root, not under it, and there is no weight.
void oracle_rms_norm_f32(const float* input, float* output, size_t length, float eps) {
    float sum = input[0] * input[0];
    for (size_t i = 1; i < length; ++i) sum = sum + input[i] * input[i];
    const float variance = sum / static_cast<float>(length);
    const float rrms = 1.0f / (std::sqrt(variance) + eps);
    for (size_t i = 0; i < length; ++i) output[i] = input[i] * rrms;
}

// src/kernel/generic/complex_mul.rs:3-20: interleaved pairs (x[2j], x[2j+1]) * (r[2j], r[2j+1]).
void oracle_complex_mul_f32(const float* a, const float* b, float* out, size_t length) {
    for (size_t i = 0; i < length; i += 2) {
        const float x = a[i], y = a[i + 1], c = b[i], d = b[i + 1];
        const float e = x * c - y * d;
        const float f = x * d + y * c;
        out[i] = e;
        out[i + 1] = f;
    }
}

// src/qwen3_moe/rope.rs:7-28: freq_j = 1 / theta^(2j/dim) in f32, angle = t * freq_j, row t =
// [cos, sin] pairs.  The reference builds each entry with Complex::new(1, angle).to_polar(),
// which yields (sqrt(1 + angle^2), atan(angle)) rather than a unit phasor; the table is not
// used anywhere in that snapshot.  This restatement writes (cos angle, sin angle), the phasor
// the complex multiply needs; faithful_to_polar != 0 reproduces the reference's text.
void oracle_precompute_freqs_cis(size_t dim, size_t rows, float theta, float* out, int faithful_to_polar) {
    std::vector<float> freqs;
    for (size_t x = 0; x < dim; x += 2) {
        const float p = static_cast<float>(x) / static_cast<float>(dim);
        freqs.push_back(1.0f / std::pow(theta, p));
    }
    for (size_t t = 0; t < rows; ++t)
        for (size_t j = 0; j < freqs.size(); ++j) {
            const float angle = static_cast<float>(t) * freqs[j];
            float* o = out + (t * freqs.size() + j) * 2;
            if (faithful_to_polar) {
                o[0] = std::sqrt(1.0f + angle * angle);
                o[1] = std::atan2(angle, 1.0f);
            } else {
                o[0] = std::cos(angle);
                o[1] = std::sin(angle);
            }
        }
}

// The finalize step of the fused QKV projection (src/kernel/x86_64/f16_512/
// matmul_rms_complex.rs:76-96: RMSNorm then RoPE on every 128-wide head of Q and K, in place)
// followed by the write of K and V into the cache at the chunk's positions (output_to_kv,
// src/compiler/zip_map/complex_zip.rs:92-98).  The rope row of chunk row h is position + h
// (complex_zip.rs:100,126).  q_weight / k_weight (may be NULL = the reference's weight-free
// norm) multiply the normalised head before the rotation.  bf16 in, fp32 arithmetic, bf16 out.
void oracle_qk_norm_rope_append_bf16(const uint16_t* q_in, const uint16_t* k_in, const uint16_t* v_in,
                                     uint16_t* q_out, uint16_t* k_cache, uint16_t* v_cache,
                                     const float* q_weight, const float* k_weight, const float* rope,
                                     const size_t* kv_strides, size_t max_batch, size_t q_heads,
                                     size_t kv_heads, size_t head_size, size_t position_index,
                                     const int32_t* positions, size_t position_interval, size_t batch_size,
                                     float eps) {
    const size_t D = head_size;
    std::vector<float> x(D), y(D);
    auto head = [&](const uint16_t* src, const float* w, const float* rope_row, uint16_t* dst, size_t dst_stride) {
        for (size_t c = 0; c < D; ++c) x[c] = bf16_to_f32(src[c]);
        oracle_rms_norm_f32(x.data(), y.data(), D, eps);
        if (w)
            for (size_t c = 0; c < D; ++c) y[c] = y[c] * w[c];
        oracle_complex_mul_f32(y.data(), rope_row, x.data(), D);
        for (size_t c = 0; c < D; ++c) dst[c * dst_stride] = f32_to_bf16(x[c]);
    };
    for (size_t h = 0; h < position_interval; ++h)
        for (size_t b = 0; b < batch_size; ++b) {
            const size_t pos = (positions ? static_cast<size_t>(positions[b]) : position_index) + h;
            const float* rope_row = rope + pos * D;
            for (size_t qh = 0; qh < q_heads; ++qh) {
                const size_t off = ((h * max_batch + b) * q_heads + qh) * D;
                head(q_in + off, q_weight, rope_row, q_out + off, 1);
            }
            for (size_t kvh = 0; kvh < kv_heads; ++kvh) {
                const size_t off = ((h * max_batch + b) * kv_heads + kvh) * D;
                const size_t dst = b * kv_strides[0] + kvh * kv_strides[1] + pos * kv_strides[2];
                head(k_in + off, k_weight, rope_row, k_cache + dst, kv_strides[3]);
                for (size_t c = 0; c < D; ++c) v_cache[dst + c * kv_strides[3]] = v_in[off + c];
            }
        }
}

// C = (residual +) A . W_nt^T, the arithmetic of the reference's projection operators
// (src/compiler/mul/matmul_add.rs:128-232: tile <- residual, then tile += A x B over the k blocks;
// src/compiler/mul/matmul3.rs:289-385 without a residual).  A is [m x k] with lda elements between
// rows, W_nt is [n x k] contiguous.  The reference accumulates in its storage type; here, as for
// attention, products and sums are fp32 (k ascending, the residual added last) and the result is
// rounded to bf16 once.  Rows are split over `threads` with assign().
void oracle_matmul_nt_bf16(const uint16_t* a, size_t lda, const uint16_t* w_nt, const uint16_t* residual,
                           size_t ldr, uint16_t* out, size_t ldc, size_t m, size_t n, size_t k, size_t threads) {
    if (threads == 0) threads = 1;
    std::vector<float> wf(n * k);
    for (size_t i = 0; i < n * k; ++i) wf[i] = bf16_to_f32(w_nt[i]);
    auto work = [&](size_t tid) {
        size_t begin = 0, end = 0;
        if (!oracle_assign(m, threads, tid, &begin, &end)) return;
        std::vector<float> row(k);
        for (size_t i = begin; i < end; ++i) {
            for (size_t c = 0; c < k; ++c) row[c] = bf16_to_f32(a[i * lda + c]);
            for (size_t j = 0; j < n; ++j) {
                const float* w = wf.data() + j * k;
                float acc = 0.0f;
                for (size_t c = 0; c < k; ++c) acc = acc + row[c] * w[c];
                if (residual) acc = acc + bf16_to_f32(residual[i * ldr + j]);
                out[i * ldc + j] = f32_to_bf16(acc);
            }
        }
    };
    if (threads == 1) {
        work(0);
        return;
    }
    std::vector<std::thread> pool;
    for (size_t t = 0; t < threads; ++t) pool.emplace_back(work, t);
    for (auto& t : pool) t.join();
}

uint16_t oracle_f32_to_bf16(float f) { return f32_to_bf16(f); }
float oracle_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }

}  // extern "C"
