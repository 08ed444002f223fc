// K3: log-sum-exp combine of partial attention results taken over disjoint key
// sets:  L = log sum_i exp(L_i),  O = sum_i O_i exp(L_i - L).
//
// No counterpart in the reference, which walks all keys of a row in one loop
// (src/kernel/generic/flash_attention.rs:69-88); it is what makes the key range
// splittable - across CTAs in the decode kernel, across GPUs in sequence-chunk
// sharding.  Lane = 4 consecutive head-dim columns of an output row.
#pragma once
#include "common.cuh"
#include "decode_splitkv.cuh"

namespace ellm {

template <typename OutT>
__device__ __forceinline__ void store_row4(OutT* dst, float4 v);
template <>
__device__ __forceinline__ void store_row4<float>(float* dst, float4 v) {
    *reinterpret_cast<float4*>(dst) = v;
}
template <>
__device__ __forceinline__ void store_row4<__nv_bfloat16>(__nv_bfloat16* dst, float4 v) {
    uint2 u;
    u.x = pack_bf16(v.x, v.y);
    u.y = pack_bf16(v.z, v.w);
    *reinterpret_cast<uint2*>(dst) = u;
}

// Combines the pieces the decode kernel left in its workspace.  Grid: one CTA of 4 warps per
// (sequence, query head); the warps share the row's pieces (a segment spread over many CTAs
// has many), each keeps a running (max, sum, O) and the four are combined through shared
// memory.  out: [max_batch, q_heads, 128], lse: [max_batch, q_heads].
template <typename OutT>
__global__ void __launch_bounds__(128) decode_merge_kernel(const DecodeParams p, OutT* out, float* lse) {
    // a following kernel launched as a programmatic dependent may start its own prologue now
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // under a programmatic dependent launch: wait until the decode grid's writes are visible
    // (a no-op for an ordinary launch)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float s_m[4], s_w[4];
    __shared__ float4 s_acc[4][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long row = blockIdx.x;
    const int b = static_cast<int>(row / p.q_heads), qh = static_cast<int>(row % p.q_heads);
    const int kvh = qh / p.group, g = qh % p.group, gt = g / 16, r = g % 16;
    const long long segs_per_seq = static_cast<long long>(p.kv_heads) * p.gtiles;
    const int seg_in_seq = kvh * p.gtiles + gt;
    const long long segment = b * segs_per_seq + seg_in_seq;
    const int tiles_b = p.prefix_out[b + 1] - p.prefix_out[b];
    const long long total = static_cast<long long>(p.prefix_out[p.batch]) * segs_per_seq;
    OutT* orow = out + row * kHeadDim + lane * 4;
    if (tiles_b == 0) {  // no key in range for this sequence
        if (warp == 0) {
            store_row4<OutT>(orow, make_float4(0.f, 0.f, 0.f, 0.f));
            if (lse && lane == 0) lse[row] = -INFINITY;
        }
        return;
    }
    const long long t0 = static_cast<long long>(p.prefix_out[b]) * segs_per_seq +
                         static_cast<long long>(seg_in_seq) * tiles_b;
    const long long c_first = cta_of_tile(total, p.num_ctas, t0);
    const long long c_last = cta_of_tile(total, p.num_ctas, t0 + tiles_b - 1);
    float m = -INFINITY, wsum = 0.0f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long c = c_first + warp; c <= c_last; c += 4) {
        const long long slot = c + segment;
        const float l = p.part_lse[slot * 16 + r];
        const float4 x = *reinterpret_cast<const float4*>(p.part_o + (slot * 16 + r) * kHeadDim + lane * 4);
        const float mn = fmaxf(m, l);
        const float a = __expf(m - mn), w = __expf(l - mn);   // m = -inf on the first piece: a = 0
        wsum = wsum * a + w;
        acc.x = acc.x * a + w * x.x; acc.y = acc.y * a + w * x.y;
        acc.z = acc.z * a + w * x.z; acc.w = acc.w * a + w * x.w;
        m = mn;
    }
    if (lane == 0) { s_m[warp] = m; s_w[warp] = wsum; }
    s_acc[warp][lane] = acc;
    __syncthreads();
    if (warp == 0) {
        float mm = fmaxf(fmaxf(s_m[0], s_m[1]), fmaxf(s_m[2], s_m[3]));
        float tot = 0.0f;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w4 = 0; w4 < 4; ++w4) {
            if (s_m[w4] == -INFINITY) continue;   // this warp had no piece
            const float a = __expf(s_m[w4] - mm);
            const float4 x = s_acc[w4][lane];
            tot += a * s_w[w4];
            o.x += a * x.x; o.y += a * x.y; o.z += a * x.z; o.w += a * x.w;
        }
        const float inv = 1.0f / tot;
        o.x *= inv; o.y *= inv; o.z *= inv; o.w *= inv;
        store_row4<OutT>(orow, o);
        if (lse && lane == 0) lse[row] = mm + __logf(tot);
    }
}

// Generic form behind ellm_attn_merge_partials: o_parts [parts, rows, 128] fp32,
// lse_parts [parts, rows].  A part whose LSE is -inf (it saw no key) weighs 0.
template <typename OutT>
__global__ void __launch_bounds__(128) merge_partials_kernel(const float* __restrict__ o_parts,
                                                             const float* __restrict__ lse_parts,
                                                             int parts, long long rows, OutT* out,
                                                             float* lse) {
    const int lane = threadIdx.x & 31;
    const long long row = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    float mmax = -INFINITY;
    for (int i = 0; i < parts; ++i) mmax = fmaxf(mmax, lse_parts[i * rows + row]);
    OutT* orow = out + row * kHeadDim + lane * 4;
    if (mmax == -INFINITY) {
        store_row4<OutT>(orow, make_float4(0.f, 0.f, 0.f, 0.f));
        if (lse && lane == 0) lse[row] = -INFINITY;
        return;
    }
    float wsum = 0.0f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = 0; i < parts; ++i) {
        const float l = lse_parts[i * rows + row];
        if (l == -INFINITY) continue;
        const float w = expf(l - mmax);
        const float4 x = *reinterpret_cast<const float4*>(o_parts + (i * rows + row) * kHeadDim + lane * 4);
        wsum += w;
        acc.x += w * x.x; acc.y += w * x.y; acc.z += w * x.z; acc.w += w * x.w;
    }
    const float inv = 1.0f / wsum;
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    store_row4<OutT>(orow, acc);
    if (lse && lane == 0) lse[row] = mmax + logf(wsum);
}

}  // namespace ellm
