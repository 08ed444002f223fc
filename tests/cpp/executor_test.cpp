// Drives the C++ host mirror (include/ellm_attention.hpp) the way the reference's executor
// drives its operator queue: pinned threads, every thread calls run(), spin barrier after each
// operator; the prompt goes in chunks, then single-token decode steps.  The result of every
// step is compared with the CPU oracle run over the whole sequence at once.
//
// Exit code 0 = parity within tolerance; prints the worst deviations.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <vector>

#include <cuda_runtime.h>

#include "ellm_attention.hpp"
#include "ellm_oracle.h"

struct AnyOp {  // the reference's Operator enum, reduced to what the test needs
    std::function<void(size_t, size_t, size_t, size_t, size_t)> f;
    void run(size_t position_index, size_t position_interval, size_t batch_size, size_t cpu_num, size_t thread_id) {
        f(position_index, position_interval, batch_size, cpu_num, thread_id);
    }
};

#define CUDA_OK(x)                                                           \
    do {                                                                     \
        cudaError_t e_ = (x);                                                \
        if (e_ != cudaSuccess) {                                             \
            std::fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_));    \
            return 2;                                                        \
        }                                                                    \
    } while (0)

int main(int argc, char** argv) {
    const size_t threads = argc > 1 ? std::strtoul(argv[1], nullptr, 10) : 6;
    const size_t B = 2, Hq = 8, Hkv = 2, D = 128, prompt = 200, chunk = 64, decode = 5, max_seq = 256;
    const size_t T = prompt + decode;
    const float scale = 1.0f / std::sqrt(128.0f);

    // seeded inputs: a small LCG mapped to roughly N(0,1) by summing 4 uniforms
    uint64_t state = 0x9E3779B97F4A7C15ull;
    auto next = [&]() {
        float s = 0.0f;
        for (int i = 0; i < 4; ++i) {
            state = state * 6364136223846793005ull + 1442695040888963407ull;
            s += static_cast<float>((state >> 40) & 0xFFFFFF) / 16777216.0f;
        }
        return (s - 2.0f) * 1.7320508f;
    };
    std::vector<uint16_t> q(T * B * Hq * D), kn(T * B * Hkv * D), vn(T * B * Hkv * D);
    for (auto& x : q) x = oracle_f32_to_bf16(next());
    for (auto& x : kn) x = oracle_f32_to_bf16(next());
    for (auto& x : vn) x = oracle_f32_to_bf16(next());

    // oracle: the whole sequence in one step against a cache filled by its own append
    const size_t strides[4] = {Hkv * max_seq * D, max_seq * D, D, 1};
    std::vector<uint16_t> ck(B * Hkv * max_seq * D, 0x7FC0 /* NaN */), cv(ck);
    oracle_kv_append_bf16(ck.data(), kn.data(), strides, B, Hkv, D, 0, T, B, nullptr);
    oracle_kv_append_bf16(cv.data(), vn.data(), strides, B, Hkv, D, 0, T, B, nullptr);
    std::vector<uint16_t> want_o(q.size());
    std::vector<float> want_l(T * B * Hq);
    oracle_attn_desc od{};
    od.q = q.data(); od.k = ck.data(); od.v = cv.data(); od.out = want_o.data(); od.lse = want_l.data();
    od.max_batch = B; od.q_heads = Hq; od.kv_heads = Hkv; od.head_size = D; od.scale = scale;
    std::memcpy(od.kv_strides, strides, sizeof(strides));
    oracle_attention_run_threads_bf16(&od, 0, T, B, 0);

    // device buffers (the library's allocate_init stand-in) and the operator
    void *dq, *dk, *dv, *dout, *dkn, *dvn, *dlse;
    const size_t chunk_q = chunk * B * Hq * D * 2, chunk_kv = chunk * B * Hkv * D * 2;
    ellm::check(ellm_device_alloc(0, chunk_q, &dq));
    ellm::check(ellm_device_alloc(0, chunk_q, &dout));
    ellm::check(ellm_device_alloc(0, chunk_kv, &dkn));
    ellm::check(ellm_device_alloc(0, chunk_kv, &dvn));
    ellm::check(ellm_device_alloc(0, chunk * B * Hq * 4, &dlse));
    ellm::check(ellm_device_alloc(0, ck.size() * 2, &dk));
    ellm::check(ellm_device_alloc(0, cv.size() * 2, &dv));
    ellm::DeviceOptions opt;
    opt.max_seq = max_seq; opt.max_interval = chunk; opt.lse = static_cast<float*>(dlse);
    opt.k_new = dkn; opt.v_new = dvn;
    auto attention = ellm::Attention<uint16_t>::make(static_cast<uint16_t*>(dq), static_cast<uint16_t*>(dk),
                                                     static_cast<uint16_t*>(dv), static_cast<uint16_t*>(dout), B, Hq, Hkv, D,
                                                     {strides[0], strides[1], strides[2], strides[3]}, scale, opt);

    std::vector<uint16_t> got_o(q.size());
    std::vector<float> got_l(T * B * Hq);
    int cuda_failures = 0;
    std::vector<AnyOp> queue;
    queue.push_back({[&](size_t p, size_t n, size_t b, size_t c, size_t t) { attention.run(p, n, b, c, t); }});
    queue.push_back({[&](size_t p, size_t n, size_t, size_t, size_t t) {  // "next operator": fetch the step's result
        if (t != 0) return;
        if (cudaMemcpy(&got_o[p * B * Hq * D], dout, n * B * Hq * D * 2, cudaMemcpyDeviceToHost) != cudaSuccess) ++cuda_failures;
        if (cudaMemcpy(&got_l[p * B * Hq], dlse, n * B * Hq * 4, cudaMemcpyDeviceToHost) != cudaSuccess) ++cuda_failures;
    }});
    auto before_step = [&](size_t p, size_t n) {  // stage the step's activations
        if (cudaMemcpy(dq, &q[p * B * Hq * D], n * B * Hq * D * 2, cudaMemcpyHostToDevice) != cudaSuccess) ++cuda_failures;
        if (cudaMemcpy(dkn, &kn[p * B * Hkv * D], n * B * Hkv * D * 2, cudaMemcpyHostToDevice) != cudaSuccess) ++cuda_failures;
        if (cudaMemcpy(dvn, &vn[p * B * Hkv * D], n * B * Hkv * D * 2, cudaMemcpyHostToDevice) != cudaSuccess) ++cuda_failures;
    };
    ellm::start_generation(queue, prompt, chunk, decode, B, before_step, threads);
    if (cuda_failures) { std::fprintf(stderr, "%d cudaMemcpy failures\n", cuda_failures); return 2; }

    double worst_o = 0, sum_o = 0, worst_l = 0;
    for (size_t i = 0; i < q.size(); ++i) {
        const double d = std::fabs(oracle_bf16_to_f32(got_o[i]) - oracle_bf16_to_f32(want_o[i]));
        if (!(d == d)) { std::fprintf(stderr, "NaN at %zu\n", i); return 1; }
        worst_o = std::max(worst_o, d);
        sum_o += d;
    }
    for (size_t i = 0; i < got_l.size(); ++i) worst_l = std::max(worst_l, static_cast<double>(std::fabs(got_l[i] - want_l[i])));
    std::vector<uint16_t> gk(ck.size());
    CUDA_OK(cudaMemcpy(gk.data(), dk, gk.size() * 2, cudaMemcpyDeviceToHost));
    size_t cache_mismatch = 0;  // rows [0, T) must equal the oracle's append bit for bit
    for (size_t b = 0; b < B; ++b)
        for (size_t h = 0; h < Hkv; ++h)
            if (std::memcmp(&gk[b * strides[0] + h * strides[1]], &ck[b * strides[0] + h * strides[1]], T * D * 2)) ++cache_mismatch;
    std::printf("threads %zu steps %zu  O max-abs %.4g mean-abs %.4g  LSE max-abs %.4g  cache mismatches %zu\n", threads,
                (prompt + chunk - 1) / chunk + decode, worst_o, sum_o / q.size(), worst_l, cache_mismatch);
    const bool ok = worst_o <= 2e-2 && sum_o / q.size() <= 2e-3 && worst_l <= 1e-3 && cache_mismatch == 0;

    // ellm::start: the live executor's fixed (0, 1) stepping also runs (every thread id calls run)
    std::vector<AnyOp> q2;
    q2.push_back({[&](size_t p, size_t n, size_t b, size_t c, size_t t) { attention.run(p, n, b, c, t); }});
    ellm::start(q2, 3, B, threads);
    return ok ? 0 : 1;
}
