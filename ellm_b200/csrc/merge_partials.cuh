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

// Combines the pieces the decode kernel left in its workspace.  Grid: one CTA per (sequence, query
// head).  A segment spread over many CTAs has many pieces (a single long sequence: one per CTA of
// the decode grid), so the combine is laid out for latency: first every thread fetches the
// log-sum-exp of one piece and the CTA agrees on their maximum, which fixes every piece's weight;
// then the warps take the pieces round-robin, kAhead loads in flight each, with no dependence
// between pieces - and the rows are requested before the weights are known; last the warps'
// partial rows are added through shared memory.
//
// Two shapes.  kWarps = 8, kAhead = 10: few rows with many pieces each (one sequence: 74 pieces per
// row).  kWarps = 2, kAhead = 4 with all tables in a few hundred bytes of dynamic shared memory: many
// rows with few pieces each (a batch) - small enough in registers and shared memory to sit on an
// SM beside two CTAs of the decode kernel, so that the whole grid is resident (and has let its own
// dependents go) long before the decode grid ends, and the next step's decode CTAs can move in as
// this step's leave instead of queueing behind this grid.
// out: [max_batch, q_heads, 128], lse: [max_batch, q_heads].
constexpr int kMergeThreads = 256;      // the wide shape
constexpr int kMergeLightThreads = 64;  // the light shape
constexpr int kMergeMaxPieces = 1024;   // weights kept in shared memory; more pieces are handled in rounds

// dynamic shared memory of the merge: tile prefix table, lengths, piece weights
__host__ __device__ inline size_t merge_smem_bytes(int batch, int pieces_cap) {
    return (static_cast<size_t>(2 * batch + 1) + static_cast<size_t>(pieces_cap)) * 4;
}

template <typename OutT, int kWarps, int kAhead>
// (both shapes are held to 64 registers: they have to fit beside two decode CTAs of ~184 registers x 128 threads -
// one wide CTA, or the light shape's three or four per SM - or they cannot move in, and release their own
// dependents, before the decode grid has drained)
__global__ void __launch_bounds__(kWarps * 32, kWarps >= 8 ? 4 : 20) decode_merge_kernel(const DecodeParams p, OutT* out, float* lse, int pieces_cap) {
    // a following kernel launched as a programmatic dependent may start its own prologue now
    ChainTrace ct(3);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ __align__(16) unsigned char merge_smem[];
    int* s_prefix = reinterpret_cast<int*>(merge_smem);                // [batch + 1]
    int* s_lens = s_prefix + p.batch + 1;                              // [batch]
    float* s_l = reinterpret_cast<float*>(s_lens + p.batch);           // [pieces_cap]
    __shared__ float s_red[kWarps];
    __shared__ float4 s_acc[kWarps][32];
    constexpr int kThreads = kWarps * 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // Where this row's pieces are follows from the positions alone, which are older than the decode
    // grid (it lets this grid start only after its own wait): the tile table is rebuilt here, before
    // the wait for the decode grid's results, instead of being read from it afterwards.
    dec_build_prefix(p, s_prefix, s_lens);
    const long long row = blockIdx.x;
    const int b = static_cast<int>(row / p.q_heads), qh = static_cast<int>(row % p.q_heads);
    const int kvh = qh / p.group, g = qh % p.group, gt = g / 16, r = g % 16;
    const long long segs_per_seq = static_cast<long long>(p.kv_heads) * p.gtiles;
    const int seg_in_seq = kvh * p.gtiles + gt;
    const long long segment = b * segs_per_seq + seg_in_seq;
    const int tiles_b = s_prefix[b + 1] - s_prefix[b];
    const long long total = static_cast<long long>(s_prefix[p.batch]) * segs_per_seq;
    OutT* orow = out + row * kHeadDim + lane * 4;
    long long c_first = 0, c_last = -1;
    if (tiles_b > 0) {
        const long long t0 = static_cast<long long>(s_prefix[b]) * segs_per_seq + static_cast<long long>(seg_in_seq) * tiles_b;
        if (dec_split_is_aligned(p, s_prefix, segs_per_seq, total)) {
            // the decode grid snapped its CTA boundaries to the segments: this segment's CTAs, of which
            // the first min(CTAs, tiles) have a piece
            c_first = dec_snap(t0, total, p.num_ctas);
            const long long n = dec_snap(t0 + tiles_b, total, p.num_ctas) - c_first;
            c_last = c_first + (n < tiles_b ? n : tiles_b) - 1;
        } else {
            c_first = cta_of_tile(total, p.num_ctas, t0);
            c_last = cta_of_tile(total, p.num_ctas, t0 + tiles_b - 1);
        }
    }
    const int pieces = static_cast<int>(c_last - c_first + 1);
    const float* lse_base = p.part_lse + (c_first + segment) * 16 + r;            // piece i at + i * 16
    const float* o_base = p.part_o + ((c_first + segment) * 16 + r) * kHeadDim + lane * 4;   // piece i at + i * 16 * 128
    // under a programmatic dependent launch: wait until the decode grid's writes are visible
    // (a no-op for an ordinary launch)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    ct.waited();
    if (tiles_b == 0) {  // no key in range for this sequence
        if (warp == 0) {
            store_row4<OutT>(orow, make_float4(0.f, 0.f, 0.f, 0.f));
            if (lse && lane == 0) lse[row] = -INFINITY;
        }
        return;
    }

    // The pieces' rows do not depend on their weights, so a warp requests the rows of its first
    // kAhead pieces before anything else: they travel while the log-sum-exps are fetched and
    // their maximum is agreed on - two dependent round trips to L2 in all instead of four or five.
    float4 x[kAhead];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
        const int i = warp + u * kWarps;
        x[u] = i < pieces ? *reinterpret_cast<const float4*>(o_base + static_cast<long long>(i) * 16 * kHeadDim)
                          : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // 1. the maximum of the pieces' log-sum-exps (every piece has seen at least one key: finite)
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < pieces; i += kThreads) {
        const float l = lse_base[static_cast<long long>(i) * 16];
        if (i < pieces_cap) s_l[i] = l;
        mx = fmaxf(mx, l);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) s_red[warp] = mx;
    __syncthreads();
    float mm = s_red[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) mm = fmaxf(mm, s_red[w]);

    // 2. weighted sums, pieces round-robin over the warps
    float wsum = 0.0f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    auto piece_lse = [&](int i) { return i < pieces_cap ? s_l[i] : lse_base[static_cast<long long>(i) * 16]; };
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
        const int i = warp + u * kWarps;
        if (i < pieces) {
            const float w = __expf(piece_lse(i) - mm);
            wsum += w;
            acc.x += w * x[u].x; acc.y += w * x[u].y; acc.z += w * x[u].z; acc.w += w * x[u].w;
        }
    }
    for (int i = warp + kAhead * kWarps; i < pieces; i += kWarps) {   // more pieces than the warps hold ahead
        const float4 y = *reinterpret_cast<const float4*>(o_base + static_cast<long long>(i) * 16 * kHeadDim);
        const float w = __expf(piece_lse(i) - mm);
        wsum += w;
        acc.x += w * y.x; acc.y += w * y.y; acc.z += w * y.z; acc.w += w * y.w;
    }
    ct.mid();   // (trace) the weighted sums are done
    s_acc[warp][lane] = acc;
    __syncthreads();   // also: every read of s_red above is done
    if (lane == 0) s_red[warp] = wsum;
    __syncthreads();

    // 3. the warps' partial rows
    if (warp == 0) {
        float tot = 0.0f;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w8 = 0; w8 < kWarps; ++w8) {
            const float4 xw = s_acc[w8][lane];
            tot += s_red[w8];
            o.x += xw.x; o.y += xw.y; o.z += xw.z; o.w += xw.w;
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

// The same combine over parts that live in separate buffers (each [rows, 128] fp32 with its
// [rows] log-sum-exps): the partials of a sharded sequence as they were computed or received,
// combined where they lie instead of being gathered into one array first.
constexpr int kMergeListMax = 16;
struct MergeList {
    const float* o[kMergeListMax];
    const float* lse[kMergeListMax];
    int parts;
};

template <typename OutT>
__global__ void __launch_bounds__(128) merge_partials_list_kernel(const MergeList m, long long rows, OutT* out, float* lse) {
    const int lane = threadIdx.x & 31;
    const long long row = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    float l[kMergeListMax];
    float mmax = -INFINITY;
#pragma unroll
    for (int i = 0; i < kMergeListMax; ++i) {
        l[i] = i < m.parts ? m.lse[i][row] : -INFINITY;
        mmax = fmaxf(mmax, l[i]);
    }
    OutT* orow = out + row * kHeadDim + lane * 4;
    if (mmax == -INFINITY) {
        store_row4<OutT>(orow, make_float4(0.f, 0.f, 0.f, 0.f));
        if (lse && lane == 0) lse[row] = -INFINITY;
        return;
    }
    float wsum = 0.0f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < kMergeListMax; ++i) {
        if (i < m.parts && l[i] != -INFINITY) {
            const float w = expf(l[i] - mmax);
            const float4 x = *reinterpret_cast<const float4*>(m.o[i] + row * kHeadDim + lane * 4);
            wsum += w;
            acc.x += w * x.x; acc.y += w * x.y; acc.z += w * x.z; acc.w += w * x.w;
        }
    }
    const float inv = 1.0f / wsum;
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    store_row4<OutT>(orow, acc);
    if (lse && lane == 0) lse[row] = mmax + logf(wsum);
}

}  // namespace ellm
