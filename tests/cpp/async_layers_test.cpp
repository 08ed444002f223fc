// Several attention-only decoder layers driven through the C++ host mirror's asynchronous executor:
// every operator enqueues on one stream (no host barrier per operator, one wait per step), the
// prompt goes in chunks, and the decode steps run either operator by operator or as one CUDA
// graph captured from the operator queue and replayed per step with the positions advanced on the
// device.  Both ways must give the same bits, and both are compared with the CPU oracle run over
// the whole sequence at once, layer after layer.
//
//   async_layers_test [threads] [layers] [decode steps]
// Exit code 0 = within tolerance; prints the worst deviations.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include <cuda_runtime.h>

#include "ellm_attention.hpp"
#include "ellm_oracle.h"

int main(int argc, char** argv) {
    const size_t threads = argc > 1 ? std::strtoul(argv[1], nullptr, 10) : 3;
    const size_t layers = argc > 2 ? std::strtoul(argv[2], nullptr, 10) : 8;
    const size_t decode = argc > 3 ? std::strtoul(argv[3], nullptr, 10) : 32;
    const size_t B = 2, Hq = 4, Hkv = 2, D = 128, hidden = 256, prompt = 80, chunk = 32, max_seq = 128;
    const size_t T = prompt + decode, Nq = Hq * D, Nkv = Hkv * D, rows = T * B, Nqkv = Nq + 2 * Nkv;
    const float scale = 1.0f / std::sqrt(128.0f), eps = 1e-6f;
    if (T > max_seq) { std::fprintf(stderr, "prompt + decode exceeds %zu\n", max_seq); return 2; }

    uint64_t state = 0x9E3779B97F4A7C15ull;
    auto next = [&]() {
        float s = 0.0f;
        for (int i = 0; i < 4; ++i) {
            state = state * 6364136223846793005ull + 1442695040888963407ull;
            s += static_cast<float>((state >> 40) & 0xFFFFFF) / 16777216.0f;
        }
        return (s - 2.0f) * 1.7320508f;
    };
    std::vector<uint16_t> x0(rows * hidden), wqkv(layers * Nqkv * hidden), wo(layers * hidden * Nq);
    for (auto& v : x0) v = oracle_f32_to_bf16(next());
    for (auto& v : wqkv) v = oracle_f32_to_bf16(next() * 0.06f);
    for (auto& v : wo) v = oracle_f32_to_bf16(next() * 0.02f);
    std::vector<float> qw(layers * D), kw(layers * D), rope(max_seq * D);
    for (auto& v : qw) v = 1.0f + 0.02f * next();
    for (auto& v : kw) v = 1.0f + 0.02f * next();
    oracle_precompute_freqs_cis(D, max_seq, 1e6f, rope.data(), 0);
    const size_t strides[4] = {Hkv * max_seq * D, max_seq * D, D, 1};

    // ---- oracle: every layer over the whole sequence as one chunk
    std::vector<uint16_t> want(x0);
    {
        std::vector<uint16_t> h(want.size()), pq(rows * Nq), pk(rows * Nkv), pv(rows * Nkv), qn(rows * Nq), att(rows * Nq),
            y(want.size());
        std::vector<float> a(hidden), b(hidden);
        for (size_t l = 0; l < layers; ++l) {
            const uint16_t* w = wqkv.data() + l * Nqkv * hidden;
            for (size_t r = 0; r < rows; ++r) {
                for (size_t c = 0; c < hidden; ++c) a[c] = oracle_bf16_to_f32(want[r * hidden + c]);
                oracle_rms_norm_f32(a.data(), b.data(), hidden, eps);
                for (size_t c = 0; c < hidden; ++c) h[r * hidden + c] = oracle_f32_to_bf16(b[c]);
            }
            oracle_matmul_nt_bf16(h.data(), hidden, w, nullptr, 0, pq.data(), Nq, rows, Nq, hidden, 4);
            oracle_matmul_nt_bf16(h.data(), hidden, w + Nq * hidden, nullptr, 0, pk.data(), Nkv, rows, Nkv, hidden, 4);
            oracle_matmul_nt_bf16(h.data(), hidden, w + (Nq + Nkv) * hidden, nullptr, 0, pv.data(), Nkv, rows, Nkv, hidden, 4);
            std::vector<uint16_t> ck(B * Hkv * max_seq * D, 0x7FC0 /* NaN */), cv(ck);
            oracle_qk_norm_rope_append_bf16(pq.data(), pk.data(), pv.data(), qn.data(), ck.data(), cv.data(), qw.data() + l * D,
                                            kw.data() + l * D, rope.data(), strides, B, Hq, Hkv, D, 0, nullptr, T, B, eps);
            oracle_attn_desc od{};
            od.q = qn.data(); od.k = ck.data(); od.v = cv.data(); od.out = att.data();
            od.max_batch = B; od.q_heads = Hq; od.kv_heads = Hkv; od.head_size = D; od.scale = scale;
            std::memcpy(od.kv_strides, strides, sizeof(strides));
            oracle_attention_run_threads_bf16(&od, 0, T, B, 0);
            oracle_matmul_nt_bf16(att.data(), Nq, wo.data() + l * hidden * Nq, want.data(), hidden, y.data(), hidden, rows, hidden, Nq, 4);
            want.swap(y);
        }
    }

    // ---- device buffers
    auto dalloc = [](size_t bytes) {
        void* p = nullptr;
        ellm::check(ellm_device_alloc(0, bytes, &p));
        return p;
    };
    const size_t m_row = chunk * B;
    auto* dx = static_cast<uint16_t*>(dalloc(m_row * hidden * 2));
    auto* dh = static_cast<uint16_t*>(dalloc(m_row * hidden * 2));
    auto* dq = static_cast<uint16_t*>(dalloc(m_row * Nq * 2));
    auto* da = static_cast<uint16_t*>(dalloc(m_row * Nq * 2));
    auto* dwqkv = static_cast<uint16_t*>(dalloc(wqkv.size() * 2));
    auto* dwo = static_cast<uint16_t*>(dalloc(wo.size() * 2));
    auto* dqw = static_cast<float*>(dalloc(qw.size() * 4));
    auto* dkw = static_cast<float*>(dalloc(kw.size() * 4));
    auto* drope = static_cast<float*>(dalloc(rope.size() * 4));
    auto* dpos = static_cast<int32_t*>(dalloc(B * 4));
    int cuda_failures = 0;
    auto up = [&](void* dst, const void* src, size_t bytes) {
        if (cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice) != cudaSuccess) ++cuda_failures;
    };
    up(dwqkv, wqkv.data(), wqkv.size() * 2);
    up(dwo, wo.data(), wo.size() * 2);
    up(dqw, qw.data(), qw.size() * 4);
    up(dkw, kw.data(), kw.size() * 4);
    up(drope, rope.data(), rope.size() * 4);
    void* stream = nullptr;
    ellm::check(ellm_stream_create(0, &stream));

    std::vector<std::vector<uint16_t>> results;
    size_t graph_nodes_expected = layers * 4 + 1;   // per layer: projection, decode, merge, output projection; then the position update
    for (int use_graph = 0; use_graph < 2; ++use_graph) {
        ellm_kv_cache* cache_obj = nullptr;
        ellm::check(ellm_kv_cache_create(0, layers, B, Hkv, max_seq, D, &cache_obj));
        ellm::ProjectionOptions popt;
        popt.max_batch = B; popt.stream = stream; popt.async = true;
        ellm::DeviceOptions aopt;
        aopt.max_seq = max_seq; aopt.max_interval = chunk; aopt.stream = stream; aopt.async = true; aopt.early_stream = true;
        std::vector<ellm::Operator> queue;
        for (size_t l = 0; l < layers; ++l) {
            void *dk = nullptr, *dv = nullptr;
            size_t st[4];
            ellm::check(ellm_kv_cache_layer(cache_obj, l, &dk, &dv, st));
            ellm::MatMul3<uint16_t>::Cache cache{static_cast<uint16_t*>(dk), static_cast<uint16_t*>(dv), {st[0], st[1], st[2], st[3]}, max_seq};
            ellm::MatMul3<uint16_t>::Norms norms;
            norms.q_weight = dqw + l * D; norms.k_weight = dkw + l * D; norms.eps = eps;
            norms.input_norm = true; norms.input_norm_eps = eps; norms.normed_scratch = dh;
            const uint16_t* w = dwqkv + l * Nqkv * hidden;
            queue.push_back(ellm::Operator::own(ellm::MatMul3<uint16_t>::make(dx, w, dq, w + Nq * hidden, w + (Nq + Nkv) * hidden, drope,
                                                                             max_seq, D, m_row, hidden, Nq, Nkv, cache, norms, popt)));
            queue.push_back(ellm::Operator::own(ellm::Attention<uint16_t>::make(dq, static_cast<uint16_t*>(dk), static_cast<uint16_t*>(dv), da, B, Hq,
                                                                               Hkv, D, {st[0], st[1], st[2], st[3]}, scale, aopt)));
            queue.push_back(ellm::Operator::own(ellm::MatMulAdd<uint16_t>::make(da, dwo + l * hidden * Nq, dx, dx, m_row, hidden, Nq, popt)));
        }
        std::vector<uint16_t> got(x0.size());
        size_t steps = 0;
        auto before_step = [&](size_t p, size_t n) { up(dx, &x0[p * B * hidden], n * B * hidden * 2); };
        auto after_step = [&](size_t p, size_t n) {
            if (cudaMemcpy(&got[p * B * hidden], dx, n * B * hidden * 2, cudaMemcpyDeviceToHost) != cudaSuccess) ++cuda_failures;
            ++steps;
        };
        ellm::AsyncOptions opt;
        opt.stream = stream; opt.positions = dpos; opt.graph_decode = use_graph != 0;
        ellm::start_generation_async(queue, prompt, chunk, decode, B, before_step, after_step, opt, threads);
        if (cuda_failures) { std::fprintf(stderr, "%d cudaMemcpy failures\n", cuda_failures); return 2; }
        if (steps != (prompt + chunk - 1) / chunk + decode) { std::fprintf(stderr, "steps %zu\n", steps); return 1; }
        results.push_back(got);
        queue.clear();
        ellm_kv_cache_destroy(cache_obj);
    }
    (void)graph_nodes_expected;
    const bool same_bits = results[0] == results[1];
    double worst = 0, sum = 0, ref = 0;
    for (size_t i = 0; i < want.size(); ++i) {
        const double w = oracle_bf16_to_f32(want[i]), d = std::fabs(oracle_bf16_to_f32(results[1][i]) - w);
        if (!(d == d)) { std::fprintf(stderr, "NaN at %zu\n", i); return 1; }
        worst = std::max(worst, d);
        sum += d;
        ref += std::fabs(w);
    }
    std::printf("threads %zu layers %zu decode steps %zu  graph == operator-by-operator: %s  output max-abs %.4g mean-abs %.4g (mean |x| %.4g)\n",
                threads, layers, decode, same_bits ? "same bits" : "DIFFERENT", worst, sum / want.size(), ref / want.size());
    ellm_stream_destroy(0, stream);
    return (same_bits && worst <= 0.5 && sum / want.size() <= 2e-2) ? 0 : 1;
}
