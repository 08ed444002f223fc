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
//   ellm::start_generation_async(...) the same stepping with the operators enqueued on one stream,
//                                   one wait per step, decode steps replayed from a CUDA graph
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
    bool early_stream = false;     // "decode_early_stream" of ellm_attn_set_option: the caller vouches that the
                                   // kernel before a decode step writes only Q and each sequence's newest cache row
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
        if (opt.early_stream) check(ellm_attn_set_option(a.handle_, "decode_early_stream", 1));
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

    // Extension: sequence b starts its chunk at positions[b] (device int32[batch_size]).
    void run_ragged(const int32_t* positions, size_t position_interval, size_t batch_size, size_t cpu_num,
                    size_t thread_id) const {
        check(ellm_attn_run_ragged(handle_, positions, position_interval, batch_size, cpu_num, thread_id));
    }
    // For async operators: waits for the stream and throws if a device-side wait ran out since the last check.
    void check_device() const { check(ellm_attn_check(handle_)); }

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
    void run_ragged(const int32_t* positions, size_t position_interval, size_t batch_size, size_t cpu_num,
                    size_t thread_id) const {
        check(ellm_matmul3_run_ragged(handle_, positions, position_interval, batch_size, cpu_num, thread_id));
    }
    void check_device() const { check(ellm_matmul_check(handle_, 0)); }

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
    // the product does not depend on the positions: the same rows as run()
    void run_ragged(const int32_t*, size_t position_interval, size_t batch_size, size_t cpu_num, size_t thread_id) const {
        run(0, position_interval, batch_size, cpu_num, thread_id);
    }
    void check_device() const { check(ellm_matmul_check(handle_, 1)); }

  private:
    MatMulAdd() = default;
    ellm_matmul_add* handle_ = nullptr;
};

// One entry of the executor's operator queue: any operator behind the common run() signature
// (the reference's enum Operator<T> dispatches to the variant's run, src/compiler/operator.rs:68-75).
class Operator {
  public:
    using Run = std::function<void(size_t, size_t, size_t, size_t, size_t)>;
    using RunRagged = std::function<void(const int32_t*, size_t, size_t, size_t, size_t)>;
    using Check = std::function<void()>;
    explicit Operator(Run run) : run_(std::move(run)) {}
    // takes ownership of an operator object with a run(position_index, position_interval, batch, cpus, tid);
    // the device operators of this header also bring run_ragged (positions in device memory) and
    // check_device, which the asynchronous executor below needs
    template <class Op>
    static Operator own(Op&& op) {
        auto held = std::make_shared<std::decay_t<Op>>(std::forward<Op>(op));
        Operator o([held](size_t p, size_t n, size_t b, size_t c, size_t t) { held->run(p, n, b, c, t); });
        o.run_ragged_ = [held](const int32_t* pos, size_t n, size_t b, size_t c, size_t t) { held->run_ragged(pos, n, b, c, t); };
        o.check_ = [held] { held->check_device(); };
        return o;
    }
    void run(size_t position_index, size_t position_interval, size_t batch_size, size_t cpu_num, size_t thread_id) const {
        run_(position_index, position_interval, batch_size, cpu_num, thread_id);
    }
    bool device_operator() const { return static_cast<bool>(run_ragged_); }
    void run_ragged(const int32_t* positions, size_t position_interval, size_t batch_size, size_t cpu_num,
                    size_t thread_id) const {
        if (!run_ragged_) throw std::logic_error("this operator has no form with positions in device memory");
        run_ragged_(positions, position_interval, batch_size, cpu_num, thread_id);
    }
    void check_device() const {
        if (check_) check_();
    }

  private:
    Run run_;
    RunRagged run_ragged_;
    Check check_;
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

// What the asynchronous executor needs: the one stream every operator of the queue was created on
// (ellm_stream_create, async = true in the operators' options) and, for graph decode, a device
// array of `batch_size` int32 positions (ellm_device_alloc) that it owns while it runs.
struct AsyncOptions {
    int device = 0;
    void* stream = nullptr;
    int32_t* positions = nullptr;   // device int32[batch_size]; required for graph_decode
    bool graph_decode = true;       // decode steps: capture the operator queue once, replay it per step
    size_t start_position = 0;      // tokens already in the cache: the first step starts here
    size_t check_every = 64;        // decode steps between two status checks of all operators (each check
                                    // reads a word back from the device per operator; a device-side wait
                                    // that ran out took seconds, so it is reported soon enough); prompt
                                    // chunks and the last step are always checked
};

// start_generation without a host barrier per operator.  The operators only enqueue on one stream
// (in queue order, by thread 0; the other threads' run() calls return at once, as always), and the
// threads meet ONE barrier per step, after thread 0 has waited for the stream and checked every
// operator's device status - in place of the barrier after each operator of
// src/serving/start.rs:69-73.  With graph_decode the first decode step runs like that (it also
// warms every kernel up), then one step's operator queue - every operator in its run_ragged form,
// reading the sequences' positions from opt.positions, followed by the update positions += 1 - is
// captured into a CUDA graph, and every further decode step is one launch of that graph.
// before_step(position, interval) runs on thread 0 before a step is enqueued (stage the step's
// input), after_step(position, interval) on thread 0 after the step's wait (fetch its output).
// Every operator of the queue must be a device operator (Operator::own of this header's classes).
template <class Op, class BeforeStep, class AfterStep>
void start_generation_async(std::vector<Op>& operator_queue, size_t prompt_length, size_t sequence_chunk_size,
                            size_t decode_steps, size_t batch_size, BeforeStep before_step, AfterStep after_step,
                            const AsyncOptions& opt, size_t thread_num = 0) {
    if (!opt.stream) throw std::invalid_argument("start_generation_async needs a stream from ellm_stream_create");
    const bool use_graph = opt.graph_decode && decode_steps > 1;
    if (use_graph && !opt.positions) throw std::invalid_argument("graph decode needs AsyncOptions::positions");
    for (auto& op : operator_queue)
        if (!op.device_operator()) throw std::invalid_argument("start_generation_async: host-side operator in the queue");
    ellm_step_graph* graph = nullptr;
    try {
        detail::spmd(thread_num, [&](size_t tid, size_t threads, Barrier& barrier, std::exception_ptr& err) {
            auto guarded = [&](auto&& f) {
                try {
                    if (!err) f();
                } catch (...) {
                    err = std::current_exception();
                }
            };
            auto finish = [&](size_t position, size_t interval, bool check_status = true) {   // one wait and one barrier per step
                if (tid == 0)
                    guarded([&] {
                        check(ellm_stream_synchronize(opt.device, opt.stream));
                        if (check_status)
                            for (auto& op : operator_queue) op.check_device();
                        after_step(position, interval);
                    });
                barrier.wait();
            };
            auto due = [&](size_t s) { return s + 1 == decode_steps || opt.check_every <= 1 || (s + 1) % opt.check_every == 0; };
            auto eager_step = [&](size_t position, size_t interval, bool ragged, bool check_status = true) {
                if (tid == 0) guarded([&] { before_step(position, interval); });
                for (auto& op : operator_queue)
                    guarded([&] {
                        if (ragged) op.run_ragged(opt.positions, interval, batch_size, threads, tid);
                        else op.run(position, interval, batch_size, threads, tid);
                    });
                finish(position, interval, check_status);
            };
            size_t position = opt.start_position;
            const size_t prompt_end = opt.start_position + prompt_length;
            while (position < prompt_end) {
                const size_t interval = std::min(sequence_chunk_size, prompt_end - position);
                eager_step(position, interval, false);
                position += interval;
            }
            if (!use_graph) {
                for (size_t s = 0; s < decode_steps; ++s) eager_step(position++, 1, false, due(s));
                return;
            }
            // first decode step: enqueued operator by operator, positions taken from the device array
            if (tid == 0)
                guarded([&] { check(ellm_positions_set(opt.positions, batch_size, static_cast<int32_t>(position), 0, opt.device, opt.stream)); });
            eager_step(position++, 1, true);
            if (tid == 0)
                guarded([&] {
                    check(ellm_positions_set(opt.positions, batch_size, 1, 1, opt.device, opt.stream));
                    // record one step; nothing runs until the graph is launched
                    check(ellm_step_graph_begin(opt.device, opt.stream));
                    try {
                        for (auto& op : operator_queue) op.run_ragged(opt.positions, 1, batch_size, 1, 0);
                        check(ellm_positions_set(opt.positions, batch_size, 1, 1, opt.device, opt.stream));
                    } catch (...) {
                        ellm_step_graph* dropped = nullptr;
                        ellm_step_graph_end(opt.device, opt.stream, &dropped);
                        ellm_step_graph_destroy(dropped);
                        throw;
                    }
                    check(ellm_step_graph_end(opt.device, opt.stream, &graph));
                });
            barrier.wait();
            for (size_t s = 1; s < decode_steps; ++s, ++position) {
                if (tid == 0)
                    guarded([&] {
                        before_step(position, 1);
                        check(ellm_step_graph_launch(graph, opt.stream));
                    });
                finish(position, 1, due(s));
            }
        });
    } catch (...) {
        ellm_step_graph_destroy(graph);
        throw;
    }
    ellm_step_graph_destroy(graph);
}

}  // namespace ellm
