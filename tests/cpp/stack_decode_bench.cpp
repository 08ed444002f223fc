// Times the decode step of an attention-only stack driven by the C++ host mirror's asynchronous
// executor (ellm::start_generation_async): per layer MatMul3 (input norm, projections, head norms,
// RoPE and cache write inside), Attention, MatMulAdd (output projection + residual) - all layers
// captured into one CUDA graph, replayed once per step with the position advanced on the device.
// Default geometry: BASELINE configs[3] (48 layers, hidden 2048, 32 q / 4 kv heads, context 32768,
// one sequence).  Weights are synthetic (one layer's worth repeated), the cache holds zeros: the
// step's time does not depend on the values.
//
//   stack_decode_bench [layers] [context] [decode steps] [graph 0/1]
// Prints one JSON line: {"tpot_ms": ..., "layers": ..., ...}
#include <chrono>
#include <cmath>
#include <cstring>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include <cuda_runtime.h>

#include "ellm_attention.hpp"

int main(int argc, char** argv) {
    const size_t layers = argc > 1 ? std::strtoul(argv[1], nullptr, 10) : 48;
    const size_t context = argc > 2 ? std::strtoul(argv[2], nullptr, 10) : 32768;
    const size_t decode = argc > 3 ? std::strtoul(argv[3], nullptr, 10) : 256;
    const bool use_graph = argc > 4 ? std::atoi(argv[4]) != 0 : true;
    const size_t B = 1, Hq = 32, Hkv = 4, D = 128, hidden = 2048;
    const size_t Nq = Hq * D, Nkv = Hkv * D, Nqkv = Nq + 2 * Nkv, max_seq = context + decode + 8;
    const float scale = 0.08838834764831845f, eps = 1e-6f;
    try {
        auto dalloc = [](size_t bytes) {
            void* p = nullptr;
            ellm::check(ellm_device_alloc(0, bytes, &p));
            return p;
        };
        uint64_t state = 0x9E3779B97F4A7C15ull;
        auto next_bf16 = [&](float amp) {   // uniform in (-amp, amp), as bf16 bits
            state = state * 6364136223846793005ull + 1442695040888963407ull;
            const float f = (static_cast<float>((state >> 40) & 0xFFFFFF) / 8388608.0f - 1.0f) * amp;
            uint32_t u;
            std::memcpy(&u, &f, 4);
            return static_cast<uint16_t>((u + 0x7FFF + ((u >> 16) & 1)) >> 16);
        };
        std::vector<uint16_t> wqkv(Nqkv * hidden), wo(hidden * Nq), x(hidden);
        for (auto& v : wqkv) v = next_bf16(0.03f);
        for (auto& v : wo) v = next_bf16(0.03f);
        for (auto& v : x) v = next_bf16(1.0f);
        auto* dwqkv = static_cast<uint16_t*>(dalloc(layers * wqkv.size() * 2));
        auto* dwo = static_cast<uint16_t*>(dalloc(layers * wo.size() * 2));
        for (size_t l = 0; l < layers; ++l) {
            if (cudaMemcpy(dwqkv + l * wqkv.size(), wqkv.data(), wqkv.size() * 2, cudaMemcpyHostToDevice) != cudaSuccess ||
                cudaMemcpy(dwo + l * wo.size(), wo.data(), wo.size() * 2, cudaMemcpyHostToDevice) != cudaSuccess)
                throw std::runtime_error("cudaMemcpy of the weights failed");
        }
        std::vector<float> rope(max_seq * D);
        for (size_t r = 0; r < max_seq; ++r)
            for (size_t j = 0; j < D / 2; ++j) {
                const float a = static_cast<float>(r) * std::pow(1e6f, -2.0f * static_cast<float>(j) / static_cast<float>(D));
                rope[r * D + 2 * j] = std::cos(a);
                rope[r * D + 2 * j + 1] = std::sin(a);
            }
        auto* drope = static_cast<float*>(dalloc(rope.size() * 4));
        cudaMemcpy(drope, rope.data(), rope.size() * 4, cudaMemcpyHostToDevice);
        auto* dx = static_cast<uint16_t*>(dalloc(hidden * 2));
        auto* dh = static_cast<uint16_t*>(dalloc(hidden * 2));
        auto* dq = static_cast<uint16_t*>(dalloc(Nq * 2));
        auto* da = static_cast<uint16_t*>(dalloc(Nq * 2));
        auto* dpos = static_cast<int32_t*>(dalloc(B * 4));
        cudaMemcpy(dx, x.data(), hidden * 2, cudaMemcpyHostToDevice);
        void* stream = nullptr;
        ellm::check(ellm_stream_create(0, &stream));
        ellm_kv_cache* cache_obj = nullptr;
        ellm::check(ellm_kv_cache_create(0, layers, B, Hkv, max_seq, D, &cache_obj));

        ellm::ProjectionOptions popt;
        popt.max_batch = B; popt.stream = stream; popt.async = true;
        ellm::DeviceOptions aopt;
        aopt.max_seq = max_seq; aopt.max_interval = 1; aopt.stream = stream; aopt.async = true; aopt.early_stream = true;
        std::vector<ellm::Operator> queue;
        for (size_t l = 0; l < layers; ++l) {
            void *dk = nullptr, *dv = nullptr;
            size_t st[4];
            ellm::check(ellm_kv_cache_layer(cache_obj, l, &dk, &dv, st));
            ellm::MatMul3<uint16_t>::Cache cache{static_cast<uint16_t*>(dk), static_cast<uint16_t*>(dv), {st[0], st[1], st[2], st[3]}, max_seq};
            ellm::MatMul3<uint16_t>::Norms norms;
            norms.eps = eps; norms.input_norm = true; norms.input_norm_eps = eps; norms.normed_scratch = dh;
            const uint16_t* w = dwqkv + l * wqkv.size();
            queue.push_back(ellm::Operator::own(ellm::MatMul3<uint16_t>::make(dx, w, dq, w + Nq * hidden, w + (Nq + Nkv) * hidden, drope,
                                                                             max_seq, D, B, hidden, Nq, Nkv, cache, norms, popt)));
            queue.push_back(ellm::Operator::own(ellm::Attention<uint16_t>::make(dq, static_cast<uint16_t*>(dk), static_cast<uint16_t*>(dv), da, B, Hq,
                                                                               Hkv, D, {st[0], st[1], st[2], st[3]}, scale, aopt)));
            queue.push_back(ellm::Operator::own(ellm::MatMulAdd<uint16_t>::make(da, dwo + l * wo.size(), dx, dx, B, hidden, Nq, popt)));
        }
        // the first two steps (operator by operator, then the first replay) are warm-up; time the rest
        size_t steps = 0;
        std::chrono::steady_clock::time_point t0, t1;
        auto before_step = [&](size_t, size_t) {};
        auto after_step = [&](size_t, size_t) {
            ++steps;
            if (steps == 2) t0 = std::chrono::steady_clock::now();
            t1 = std::chrono::steady_clock::now();
        };
        ellm::AsyncOptions opt;
        opt.stream = stream; opt.positions = dpos; opt.graph_decode = use_graph; opt.start_position = context;
        ellm::start_generation_async(queue, 0, 1, decode, B, before_step, after_step, opt, 1);
        const double ms = std::chrono::duration<double, std::milli>(t1 - t0).count() / static_cast<double>(steps - 2);
        std::vector<uint16_t> y(hidden);
        cudaMemcpy(y.data(), dx, hidden * 2, cudaMemcpyDeviceToHost);
        bool finite = true;
        for (auto v : y) finite = finite && ((v & 0x7F80) != 0x7F80);
        const double kv_bytes = 2.0 * Hkv * D * 2 * (context + decode / 2.0) * layers, w_bytes = 2.0 * (Nqkv + Nq) * hidden * layers;
        std::printf("{\"tpot_ms\": %.5f, \"layers\": %zu, \"context\": %zu, \"decode_steps\": %zu, \"timed_steps\": %zu, \"cuda_graph\": %s, "
                    "\"decode_gbs\": %.1f, \"finite\": %s, \"timing\": \"host clock around the steps, one stream wait per step\"}\n",
                    ms, layers, context, decode, steps - 2, use_graph ? "true" : "false", (kv_bytes + w_bytes) / ms / 1e6,
                    finite ? "true" : "false");
        queue.clear();
        ellm_kv_cache_destroy(cache_obj);
        ellm_stream_destroy(0, stream);
        return finite ? 0 : 1;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "stack_decode_bench: %s\n", e.what());
        return 2;
    }
}
