// One attention-only decoder layer driven through the C++ host mirror's operator queue, the way
// the reference's executor runs its graph: MatMul3 (with the layer's input norm, the head norms,
// RoPE and the cache write inside) -> Attention -> MatMulAdd (output projection + residual), every
// pinned thread calling every operator's run() with a spin barrier after each.  The prompt goes in
// chunks (tensor-memory GEMM for full chunks, the weight-streaming kernel for the short last one),
// then single-token decode steps.  The layer output of every step is compared with the CPU oracle
// run over the whole sequence at once.
//
// Exit code 0 = within tolerance; prints the worst deviations.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include <cuda_runtime.h>

#include "ellm_attention.hpp"
#include "ellm_oracle.h"

int main(int argc, char** argv) {
    const size_t threads = argc > 1 ? std::strtoul(argv[1], nullptr, 10) : 4;
    const size_t B = 2, Hq = 4, Hkv = 2, D = 128, hidden = 256, prompt = 200, chunk = 64, decode = 5, max_seq = 256;
    const size_t T = prompt + decode, Nq = Hq * D, Nkv = Hkv * D, rows = T * B;
    const float scale = 1.0f / std::sqrt(128.0f), eps = 1e-6f;

    uint64_t state = 0x243F6A8885A308D3ull;
    auto next = [&]() {
        float s = 0.0f;
        for (int i = 0; i < 4; ++i) {
            state = state * 6364136223846793005ull + 1442695040888963407ull;
            s += static_cast<float>((state >> 40) & 0xFFFFFF) / 16777216.0f;
        }
        return (s - 2.0f) * 1.7320508f;
    };
    std::vector<uint16_t> x(rows * hidden), wqkv((Nq + 2 * Nkv) * hidden), wo(hidden * Nq);
    for (auto& v : x) v = oracle_f32_to_bf16(next());
    for (auto& v : wqkv) v = oracle_f32_to_bf16(next() * 0.06f);
    for (auto& v : wo) v = oracle_f32_to_bf16(next() * 0.04f);
    std::vector<float> qw(D), kw(D), rope(max_seq * D);
    for (auto& v : qw) v = 1.0f + 0.02f * next();
    for (auto& v : kw) v = 1.0f + 0.02f * next();
    oracle_precompute_freqs_cis(D, max_seq, 1e6f, rope.data(), 0);
    const size_t strides[4] = {Hkv * max_seq * D, max_seq * D, D, 1};

    // ---- oracle: the whole sequence as one chunk
    std::vector<uint16_t> h(x.size()), pq(rows * Nq), pk(rows * Nkv), pv(rows * Nkv), qn(rows * Nq);
    {
        std::vector<float> a(hidden), b(hidden);
        for (size_t r = 0; r < rows; ++r) {
            for (size_t c = 0; c < hidden; ++c) a[c] = oracle_bf16_to_f32(x[r * hidden + c]);
            oracle_rms_norm_f32(a.data(), b.data(), hidden, eps);
            for (size_t c = 0; c < hidden; ++c) h[r * hidden + c] = oracle_f32_to_bf16(b[c]);
        }
    }
    oracle_matmul_nt_bf16(h.data(), hidden, wqkv.data(), nullptr, 0, pq.data(), Nq, rows, Nq, hidden, 4);
    oracle_matmul_nt_bf16(h.data(), hidden, wqkv.data() + Nq * hidden, nullptr, 0, pk.data(), Nkv, rows, Nkv, hidden, 4);
    oracle_matmul_nt_bf16(h.data(), hidden, wqkv.data() + (Nq + Nkv) * hidden, nullptr, 0, pv.data(), Nkv, rows, Nkv, hidden, 4);
    std::vector<uint16_t> ck(B * Hkv * max_seq * D, 0x7FC0 /* NaN */), cv(ck);
    oracle_qk_norm_rope_append_bf16(pq.data(), pk.data(), pv.data(), qn.data(), ck.data(), cv.data(), qw.data(), kw.data(),
                                    rope.data(), strides, B, Hq, Hkv, D, 0, nullptr, T, B, eps);
    std::vector<uint16_t> att(rows * Nq), want(x.size());
    oracle_attn_desc od{};
    od.q = qn.data(); od.k = ck.data(); od.v = cv.data(); od.out = att.data();
    od.max_batch = B; od.q_heads = Hq; od.kv_heads = Hkv; od.head_size = D; od.scale = scale;
    std::memcpy(od.kv_strides, strides, sizeof(strides));
    oracle_attention_run_threads_bf16(&od, 0, T, B, 0);
    oracle_matmul_nt_bf16(att.data(), Nq, wo.data(), x.data(), hidden, want.data(), hidden, rows, hidden, Nq, 4);

    // ---- device buffers and the operator queue
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
    auto* dk = static_cast<uint16_t*>(dalloc(ck.size() * 2));
    auto* dv = static_cast<uint16_t*>(dalloc(cv.size() * 2));
    auto* dwqkv = static_cast<uint16_t*>(dalloc(wqkv.size() * 2));
    auto* dwo = static_cast<uint16_t*>(dalloc(wo.size() * 2));
    auto* dqw = static_cast<float*>(dalloc(D * 4));
    auto* dkw = static_cast<float*>(dalloc(D * 4));
    auto* drope = static_cast<float*>(dalloc(rope.size() * 4));
    int cuda_failures = 0;
    auto up = [&](void* dst, const void* src, size_t bytes) {
        if (cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice) != cudaSuccess) ++cuda_failures;
    };
    up(dwqkv, wqkv.data(), wqkv.size() * 2);
    up(dwo, wo.data(), wo.size() * 2);
    up(dqw, qw.data(), D * 4);
    up(dkw, kw.data(), D * 4);
    up(drope, rope.data(), rope.size() * 4);

    ellm::ProjectionOptions popt;
    popt.max_batch = B;
    ellm::MatMul3<uint16_t>::Cache cache{dk, dv, {strides[0], strides[1], strides[2], strides[3]}, max_seq};
    ellm::MatMul3<uint16_t>::Norms norms;
    norms.q_weight = dqw; norms.k_weight = dkw; norms.eps = eps;
    norms.input_norm = true; norms.input_norm_eps = eps; norms.normed_scratch = dh;
    ellm::DeviceOptions aopt;
    aopt.max_seq = max_seq; aopt.max_interval = chunk;
    std::vector<ellm::Operator> queue;
    queue.push_back(ellm::Operator::own(ellm::MatMul3<uint16_t>::make(dx, dwqkv, dq, dwqkv + Nq * hidden, dwqkv + (Nq + Nkv) * hidden,
                                                                     drope, max_seq, D, m_row, hidden, Nq, Nkv, cache, norms, popt)));
    queue.push_back(ellm::Operator::own(ellm::Attention<uint16_t>::make(dq, dk, dv, da, B, Hq, Hkv, D,
                                                                       {strides[0], strides[1], strides[2], strides[3]}, scale, aopt)));
    queue.push_back(ellm::Operator::own(ellm::MatMulAdd<uint16_t>::make(da, dwo, dx, dx, m_row, hidden, Nq, popt)));
    std::vector<uint16_t> got(x.size());
    queue.push_back(ellm::Operator([&](size_t p, size_t n, size_t, size_t, size_t t) {  // "next operator": fetch the layer output
        if (t == 0 && cudaMemcpy(&got[p * B * hidden], dx, n * B * hidden * 2, cudaMemcpyDeviceToHost) != cudaSuccess) ++cuda_failures;
    }));
    auto before_step = [&](size_t p, size_t n) { up(dx, &x[p * B * hidden], n * B * hidden * 2); };
    ellm::start_generation(queue, prompt, chunk, decode, B, before_step, threads);
    if (cuda_failures) { std::fprintf(stderr, "%d cudaMemcpy failures\n", cuda_failures); return 2; }

    double worst = 0, sum = 0;
    for (size_t i = 0; i < got.size(); ++i) {
        const double d = std::fabs(oracle_bf16_to_f32(got[i]) - oracle_bf16_to_f32(want[i]));
        if (!(d == d)) { std::fprintf(stderr, "NaN at %zu\n", i); return 1; }
        worst = std::max(worst, d);
        sum += d;
    }
    std::vector<uint16_t> gv(cv.size());
    if (cudaMemcpy(gv.data(), dv, gv.size() * 2, cudaMemcpyDeviceToHost) != cudaSuccess) return 2;
    // V rows are the projection of the normalised input: a normalised value may sit one bf16 step from
    // the oracle's (other summation order in the norm), which moves a projected value by a few 1e-3
    size_t v_far = 0;
    for (size_t b = 0; b < B; ++b)
        for (size_t hh = 0; hh < Hkv; ++hh)
            for (size_t i = 0; i < T * D; ++i) {
                const size_t at = b * strides[0] + hh * strides[1] + i;
                const float w = oracle_bf16_to_f32(cv[at]), g = oracle_bf16_to_f32(gv[at]);
                if (!(std::fabs(g - w) <= std::fabs(w) / 64.0f + 4e-3f)) ++v_far;
            }
    std::printf("threads %zu steps %zu  layer output max-abs %.4g mean-abs %.4g  V rows off %zu\n", threads,
                (prompt + chunk - 1) / chunk + decode, worst, sum / got.size(), v_far);
    return (worst <= 0.25 && sum / got.size() <= 1e-2 && v_far == 0) ? 0 : 1;
}
