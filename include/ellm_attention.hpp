// C++ host-side mirror of the reference's attention operator and of the executor that
// drives it, over the C ABI of ellm_attn.h.  Header-only; link against libellm_attn.so.
//
// The reference is a Rust crate; where no Rust toolchain exists this header is the host side
// a caller compiles against.  Names, argument order and meaning follow the reference:
//
//   ellm::Attention<T>::make(...)   Attention::new        src/compiler/mul/attention.rs:41-67
//   ellm::Attention<T>::run(...)    Attention::run        src/compiler/mul/attention.rs:69-76
//   ellm::MatMul3<T>::make / run    MatMul3::new / run    src/compiler/mul/matmul3.rs:60-119, 289-385
//   ellm::MatMulAdd<T>::make / run  MatMulAdd::new / run  src/compiler/mul/matmul_add.rs:60-126, 128-232
//   ellm::Operator                  enum Operator<T>      src/compiler/operator.rs:30-75 (one run() for all)
//   ellm::Barrier                   runtime::barrier      src/runtime/barrier.rs:7-40
//   ellm::assign(...)               compiler::assign      src/compiler/assign.rs:11-38
//   ellm::start(...)                serving::start::start src/serving/start.rs:18-86
//   ellm::start_generation(...)     the prompt-chunk / decode stepping the reference keeps in
//                                   src/serving/start copy.rs:84-110 (not compiled there)
//
// Errors: the reference aborts (panic = "abort"); here a non-zero status becomes a
// std::runtime_error carrying ellm_last_error().
#pragma once

#include <algorithm>
#include <atomic>
#include <cstddef>
#include <cstdint>
#include <exception>
#include <functional>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <thread>
#include <utility>
#include <vector>

#include <pthread.h>
#include <sched.h>

#include "ellm_attn.h"
#include "ellm_proj.h"

namespace ellm {

inline void check(int status) {
    if (status != ELLM_OK) throw std::runtime_error(std::string("ellm_attn: ") + ellm_last_error());
}

// [0, length) split in `num` parts, the first length % num parts one longer; empty parts -> nullopt.
inline std::optional<std::pair<size_t, size_t>> assign(size_t length, size_t num, size_t id) {
    if (length < id + 1) return std::nullopt;
    const size_t q = length / num, r = length % num;
    if (id < r) return std::make_pair((q + 1) * id, (q + 1) * id + q + 1);
    return std::make_pair(q * id + r, q * id + r + q);
}

// What a device needs beyond the reference's constructor arguments.
struct DeviceOptions {
    size_t max_seq = 0;            // rows per (sequence, kv head) in the cache
    size_t max_interval = 1;       // most chunk rows one run() is given
    float* lse = nullptr;          // optional fp32 log-sum-exp output
    const void* k_new = nullptr;   // the chunk's new K/V rows, appended by run()
    const void* v_new = nullptr;
    int device = 0;
    void* stream = nullptr;        // cudaStream_t
    bool async = false;            // false: run() returns after the stream drained (barrier semantics)
    int prefill_kernel = ELLM_PREFILL_AUTO;
};

// T is the element type of the buffers; only 16-bit bf16 storage is implemented.
template <typename T>
class Attention {
    static_assert(sizeof(T) == 2, "bf16 storage (2-byte elements) only");

  public:
    // Attention::new(q_ptr, k_ptr, v_ptr, output_ptr, batch_size, attention_head_num, kv_head_num,
    //                head_size, kv_strides, inverse_sqrt_head)
    static Attention make(const T* q_ptr, const T* k_ptr, const T* v_ptr, T* output_ptr, size_t batch_size,
                          size_t attention_head_num, size_t kv_head_num, size_t head_size,
                          const std::vector<size_t>& kv_strides, float inverse_sqrt_head, const DeviceOptions& opt) {
        if (kv_strides.size() != 4) throw std::invalid_argument("kv_strides must have 4 entries");
        ellm_attn_desc d{};
        d.q = q_ptr;
        d.k_cache = const_cast<T*>(k_ptr);
        d.v_cache = const_cast<T*>(v_ptr);
        d.out = output_ptr;
        d.lse = opt.lse;
        d.k_new = opt.k_new;
        d.v_new = opt.v_new;
        d.max_batch = batch_size;
        d.q_heads = attention_head_num;
        d.kv_heads = kv_head_num;
        d.head_size = head_size;
        for (int i = 0; i < 4; ++i) d.kv_strides[i] = kv_strides[i];
        d.max_seq = opt.max_seq;
        d.max_interval = opt.max_interval;
        d.scale = inverse_sqrt_head;
        d.dtype = ELLM_DTYPE_BF16;
        d.device = opt.device;
        d.stream = opt.stream;
        d.async = opt.async ? 1 : 0;
        d.prefill_kernel = opt.prefill_kernel;
        Attention a;
        check(ellm_attn_create(&d, &a.handle_));
        return a;
    }

    Attention(Attention&& o) noexcept : handle_(o.handle_) { o.handle_ = nullptr; }
    Attention& operator=(Attention&& o) noexcept {
        if (this != &o) {
            ellm_attn_destroy(handle_);
            handle_ = o.handle_;
            o.handle_ = nullptr;
        }
        return *this;
    }
    Attention(const Attention&) = delete;
    Attention& operator=(const Attention&) = delete;
    ~Attention() { ellm_attn_destroy(handle_); }

    // Called by every worker thread, like any Operator::run (src/compiler/operator.rs:68-75).
    void run(size_t position_index, size_t position_interval, size_t batch_size, size_t cpu_num,
             size_t thread_id) const {
        check(ellm_attn_run(handle_, position_index, position_interval, batch_size, cpu_num, thread_id));
    }

    ellm_attn* handle() const { return handle_; }

  private:
    Attention() = default;
    ellm_attn* handle_ = nullptr;
};

// What the projections need beyond the reference's constructor arguments.
struct ProjectionOptions {
    size_t max_batch = 1;          // sequences per chunk row: matrix row = chunk row * max_batch + sequence
    int device = 0;
    void* stream = nullptr;
    bool async = false;
};

// The three projections of an attention block with their finalize step (per-head RMS norm, RoPE)
// and the write of K and V into the static cache.
template <typename T>
class MatMul3 {
    static_assert(sizeof(T) == 2, "bf16 storage (2-byte elements) only");

  public:
    struct Cache {                 // where K and V rows go instead of k_state_ptr / v_state_ptr
        T* k_cache = nullptr;
        T* v_cache = nullptr;
        std::vector<size_t> kv_strides;
        size_t max_seq = 0;
    };
    struct Norms {                 // optional extensions: head-norm weights, the layer's input norm
        const float* q_weight = nullptr;
        const float* k_weight = nullptr;
        float eps = 1e-6f;
        bool input_norm = false;
        float input_norm_eps = 1e-6f;
        T* normed_scratch = nullptr;
    };
    // MatMul3::new(hidden_ptr, q_weight_ptr_nt, q_state_ptr, k_weight_ptr_nt, [k_state_ptr], v_weight_ptr_nt,
    //              [v_state_ptr], rope_ptr, head_dim, m_row, col, b_q_row, b_kv_row, ...)
    static MatMul3 make(const T* hidden_ptr, const T* q_weight_ptr_nt, T* q_state_ptr, const T* k_weight_ptr_nt,
                        const T* v_weight_ptr_nt, const float* rope_ptr, size_t rope_rows, size_t head_dim, size_t m_row,
                        size_t col, size_t b_q_row, size_t b_kv_row, const Cache& cache, const Norms& norms,
                        const ProjectionOptions& opt) {
        if (cache.kv_strides.size() != 4) throw std::invalid_argument("kv_strides must have 4 entries");
        ellm_matmul3_desc d{};
        d.hidden = hidden_ptr;
        d.wq_nt = q_weight_ptr_nt;
        d.wk_nt = k_weight_ptr_nt;
        d.wv_nt = v_weight_ptr_nt;
        d.q_state = q_state_ptr;
        d.k_cache = cache.k_cache;
        d.v_cache = cache.v_cache;
        for (int i = 0; i < 4; ++i) d.kv_strides[i] = cache.kv_strides[i];
        d.rope = rope_ptr;
        d.rope_rows = rope_rows;
        d.q_norm_weight = norms.q_weight;
        d.k_norm_weight = norms.k_weight;
        d.head_dim = head_dim;
        d.m_row = m_row;
        d.col = col;
        d.b_q_row = b_q_row;
        d.b_kv_row = b_kv_row;
        d.max_batch = opt.max_batch;
        d.max_seq = cache.max_seq;
        d.eps = norms.eps;
        d.device = opt.device;
        d.stream = opt.stream;
        d.async = opt.async ? 1 : 0;
        d.input_norm = norms.input_norm ? 1 : 0;
        d.input_norm_eps = norms.input_norm_eps;
        d.normed_scratch = norms.normed_scratch;
        MatMul3 m;
        check(ellm_matmul3_create(&d, &m.handle_));
        return m;
    }
    MatMul3(MatMul3&& o) noexcept : handle_(o.handle_) { o.handle_ = nullptr; }
    MatMul3(const MatMul3&) = delete;
    MatMul3& operator=(const MatMul3&) = delete;
    ~MatMul3() { ellm_matmul3_destroy(handle_); }
    void run(size_t position_index, size_t position_interval, size_t batch_size, size_t cpu_num, size_t thread_id) const {
        check(ellm_matmul3_run(handle_, position_index, position_interval, batch_size, cpu_num, thread_id));
    }

  private:
    MatMul3() = default;
    ellm_matmul3* handle_ = nullptr;
};

// output = residual + A . W_nt^T (residual may be null: the plain MatMul).
template <typename T>
class MatMulAdd {
    static_assert(sizeof(T) == 2, "bf16 storage (2-byte elements) only");

  public:
    // MatMulAdd::new(ptr1, ptr2 (N x K), ptr3 (residual), output_ptr, m_max, n_max, k_max, ...)
    static MatMulAdd make(const T* ptr1, const T* ptr2_nt, const T* ptr3, T* output_ptr, size_t m_max, size_t n_max,
                          size_t k_max, const ProjectionOptions& opt) {
        ellm_matmul_add_desc d{};
        d.a = ptr1;
        d.w_nt = ptr2_nt;
        d.residual = ptr3;
        d.output = output_ptr;
        d.m_max = m_max;
        d.n_max = n_max;
        d.k_max = k_max;
        d.max_batch = opt.max_batch;
        d.device = opt.device;
        d.stream = opt.stream;
        d.async = opt.async ? 1 : 0;
        MatMulAdd m;
        check(ellm_matmul_add_create(&d, &m.handle_));
        return m;
    }
    MatMulAdd(MatMulAdd&& o) noexcept : handle_(o.handle_) { o.handle_ = nullptr; }
    MatMulAdd(const MatMulAdd&) = delete;
    MatMulAdd& operator=(const MatMulAdd&) = delete;
    ~MatMulAdd() { ellm_matmul_add_destroy(handle_); }
    void run(size_t position_index, size_t position_interval, size_t batch_size, size_t cpu_num, size_t thread_id) const {
        check(ellm_matmul_add_run(handle_, position_index, position_interval, batch_size, cpu_num, thread_id));
    }

  private:
    MatMulAdd() = default;
    ellm_matmul_add* handle_ = nullptr;
};

// One entry of the executor's operator queue: any operator behind the common run() signature
// (the reference's enum Operator<T> dispatches to the variant's run, src/compiler/operator.rs:68-75).
class Operator {
  public:
    using Run = std::function<void(size_t, size_t, size_t, size_t, size_t)>;
    explicit Operator(Run run) : run_(std::move(run)) {}
    // takes ownership of an operator object with a run(position_index, position_interval, batch, cpus, tid)
    template <class Op>
    static Operator own(Op&& op) {
        auto held = std::make_shared<std::decay_t<Op>>(std::forward<Op>(op));
        return Operator([held](size_t p, size_t n, size_t b, size_t c, size_t t) { held->run(p, n, b, c, t); });
    }
    void run(size_t position_index, size_t position_interval, size_t batch_size, size_t cpu_num, size_t thread_id) const {
        run_(position_index, position_interval, batch_size, cpu_num, thread_id);
    }

  private:
    Run run_;
};

// Arrival counter + generation word; waiters spin on the generation.
class Barrier {
  public:
    explicit Barrier(size_t tids) : tids_(tids) {}
    void wait() {
        const size_t gen = generation_.load(std::memory_order_relaxed);
        const size_t arrived = arrived_.fetch_add(1, std::memory_order_acq_rel) + 1;
        if (arrived == tids_) {
            arrived_.store(0, std::memory_order_relaxed);
            generation_.store(gen + 1, std::memory_order_release);
            return;
        }
        while (generation_.load(std::memory_order_acquire) == gen) {
#if defined(__x86_64__)
            __builtin_ia32_pause();
#endif
        }
    }

  private:
    alignas(64) std::atomic<size_t> arrived_{0};
    alignas(64) std::atomic<size_t> generation_{0};
    size_t tids_;
};

namespace detail {
inline void pin_to_core(size_t i) {
    cpu_set_t all;
    CPU_ZERO(&all);
    if (sched_getaffinity(0, sizeof(all), &all) != 0) return;
    const int n = CPU_COUNT(&all);
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

// Runs body(thread_id, barrier) on `thread_num` pinned threads; the first exception is rethrown
// after every thread has joined (a throwing thread keeps meeting the barrier through `failed`).
template <class Body>
void spmd(size_t thread_num, Body body) {
    if (thread_num == 0) thread_num = std::thread::hardware_concurrency();
    if (thread_num == 0) thread_num = 1;
    Barrier barrier(thread_num);
    std::vector<std::thread> pool;
    std::vector<std::exception_ptr> errors(thread_num);
    for (size_t tid = 0; tid < thread_num; ++tid)
        pool.emplace_back([&, tid] {
            pin_to_core(tid);
            body(tid, thread_num, barrier, errors[tid]);
        });
    for (auto& t : pool) t.join();
    for (auto& e : errors)
        if (e) std::rethrow_exception(e);
}
}  // namespace detail

// serving::start::start: every thread runs every operator of the queue with (0, 1, batch, threads,
// tid) and meets the barrier after each, `sequence_length` times (src/serving/start.rs:69-73).
template <class Op>
void start(std::vector<Op>& operator_queue, size_t sequence_length, size_t batch_size, size_t thread_num = 0) {
    detail::spmd(thread_num, [&](size_t tid, size_t threads, Barrier& barrier, std::exception_ptr& err) {
        for (size_t p = 0; p < sequence_length; ++p)
            for (auto& op : operator_queue) {
                try {
                    if (!err) op.run(0, 1, batch_size, threads, tid);
                } catch (...) {
                    err = std::current_exception();
                }
                barrier.wait();
            }
    });
}

// The stepping the reference intends: the prompt in chunks of `sequence_chunk_size` rows with
// run(position, chunk, ...), then `decode_steps` single-row steps with run(position, 1, ...).
// `before_step(position, interval)` runs on thread 0 before each step (e.g. to stage that step's
// activations) and is followed by a barrier so that every thread sees its effects.
template <class Op, class BeforeStep>
void start_generation(std::vector<Op>& operator_queue, size_t prompt_length, size_t sequence_chunk_size,
                      size_t decode_steps, size_t batch_size, BeforeStep before_step, size_t thread_num = 0) {
    detail::spmd(thread_num, [&](size_t tid, size_t threads, Barrier& barrier, std::exception_ptr& err) {
        auto step = [&](size_t position, size_t interval) {
            try {
                if (tid == 0 && !err) before_step(position, interval);
            } catch (...) {
                err = std::current_exception();
            }
            barrier.wait();
            for (auto& op : operator_queue) {
                try {
                    if (!err) op.run(position, interval, batch_size, threads, tid);
                } catch (...) {
                    err = std::current_exception();
                }
                barrier.wait();
            }
        };
        size_t position = 0;
        while (position < prompt_length) {
            const size_t interval = std::min(sequence_chunk_size, prompt_length - position);
            step(position, interval);
            position += interval;
        }
        for (size_t s = 0; s < decode_steps; ++s) step(position++, 1);
    });
}

}  // namespace ellm
