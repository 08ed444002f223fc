// K5: the step between the QKV projection and attention - per-head RMSNorm, interleaved
// RoPE, and the write of K and V into the static cache - in one pass over the projected rows.
//
// Replaces the finalize step of the reference's fused projection
// (matmul_finalize_rmsnorm_rope_inplace_3x128, src/kernel/x86_64/f16_512/
// matmul_rms_complex.rs:76-96: rms_norm then complex_mul on each 128-wide head of Q and K)
// and the output_to_kv write that follows it (src/compiler/zip_map/complex_zip.rs:92-98).
//   norm : y = x / (sqrt(mean x^2) + eps)          (src/kernel/generic/rms_norm.rs:6-26)
//   rope : (y[2j], y[2j+1]) * (cos, sin)[pos][j]   (src/kernel/generic/complex_mul.rs:3-20)
// An optional per-channel weight multiplies the normalised head before the rotation (the
// reference's norm has none).  HBM-bound: every projected row is read once and written once.
// One warp per head row; a lane owns 4 consecutive channels (two rotation pairs).
#pragma once
#include "common.cuh"

namespace ellm {

struct NormRopeParams {
    const __nv_bfloat16* q_in;   // row (chunk row, sequence) at q_in + row * q_in_stride, [q_heads, 128] inside
    const __nv_bfloat16* k_in;   // row at k_in + row * kv_in_stride, [kv_heads, 128] inside
    const __nv_bfloat16* v_in;
    long long q_in_stride, kv_in_stride;   // elements; q_heads*128 and kv_heads*128 when contiguous
    __nv_bfloat16* q_out;        // same layout as q_in (may alias it)
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    const float* q_weight;       // [128] or nullptr
    const float* k_weight;
    const float* rope;           // [rope_rows, 128] interleaved (cos, sin)
    const int32_t* positions;    // per-sequence chunk start or nullptr
    long long position_index;
    long long s0, s1, s2;
    long long max_seq, rope_rows;
    int interval, batch, max_batch, q_heads, kv_heads;
    float eps;
};

__global__ void __launch_bounds__(256) qk_norm_rope_append_kernel(const NormRopeParams p) {
    // programmatic dependent launches: the next kernel may be set up now; this one waits for the
    // kernel before it (the projection that wrote its input) - both no-ops for ordinary launches
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // after the wait: see proj_skinny.cuh
    const int lane = threadIdx.x & 31;
    const int heads = p.q_heads + 2 * p.kv_heads;
    const long long total = static_cast<long long>(p.interval) * p.batch * heads;
    const long long w = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= total) return;
    const int head = static_cast<int>(w % heads);
    const int b = static_cast<int>((w / heads) % p.batch);
    const int h = static_cast<int>(w / (static_cast<long long>(heads) * p.batch));
    const long long pos = (p.positions ? static_cast<long long>(p.positions[b]) : p.position_index) + h;
    const long long row = static_cast<long long>(h) * p.max_batch + b;

    if (head >= p.q_heads + p.kv_heads) {  // V: plain row copy into the cache
        const int kvh = head - p.q_heads - p.kv_heads;
        // a position without a rotation row leaves the token's whole cache line untouched (its K row
        // is skipped below for the same reason), never a new V beside a stale K
        if (pos < 0 || pos >= p.max_seq || pos >= p.rope_rows) return;
        const uint2 v = *reinterpret_cast<const uint2*>(p.v_in + row * p.kv_in_stride + kvh * kHeadDim + lane * 4);
        *reinterpret_cast<uint2*>(p.v_cache + b * p.s0 + kvh * p.s1 + pos * p.s2 + lane * 4) = v;
        return;
    }
    const bool is_q = head < p.q_heads;
    const int kvh = head - p.q_heads;
    const __nv_bfloat16* src = is_q ? p.q_in + row * p.q_in_stride + head * kHeadDim : p.k_in + row * p.kv_in_stride + kvh * kHeadDim;
    if (!is_q && (pos < 0 || pos >= p.max_seq)) return;
    if (pos < 0 || pos >= p.rope_rows) return;  // no rotation row for this position: leave the output untouched
    const uint2 raw = *reinterpret_cast<const uint2*>(src + lane * 4);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    float x[4] = {__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi)};
    float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rrms = 1.0f / (sqrtf(ss / static_cast<float>(kHeadDim)) + p.eps);
    const float* wgt = is_q ? p.q_weight : p.k_weight;
    float4 wv = make_float4(1.f, 1.f, 1.f, 1.f);
    if (wgt) wv = *reinterpret_cast<const float4*>(wgt + lane * 4);
    const float y0 = x[0] * rrms * wv.x, y1 = x[1] * rrms * wv.y, y2 = x[2] * rrms * wv.z, y3 = x[3] * rrms * wv.w;
    const float4 cs = *reinterpret_cast<const float4*>(p.rope + pos * kHeadDim + lane * 4);  // cos0 sin0 cos1 sin1
    uint2 outv;
    outv.x = pack_bf16(y0 * cs.x - y1 * cs.y, y0 * cs.y + y1 * cs.x);
    outv.y = pack_bf16(y2 * cs.z - y3 * cs.w, y2 * cs.w + y3 * cs.z);
    __nv_bfloat16* dst = is_q ? p.q_out + (row * p.q_heads + head) * kHeadDim
                              : p.k_cache + b * p.s0 + kvh * p.s1 + pos * p.s2;
    *reinterpret_cast<uint2*>(dst + lane * 4) = outv;
}

}  // namespace ellm
