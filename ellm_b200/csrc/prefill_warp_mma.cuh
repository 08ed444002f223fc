// K1 (general form): causal grouped-query flash-attention over a chunk of query
// rows on the warp-level tensor-core MMA.  It takes every shape the operator
// accepts - any chunk length, any start position, ragged per-sequence positions,
// a restricted key window, fp32 partial output.  The operator picks it by itself
// only for chunks of fewer than 16 packed rows; everything else goes to the
// tcgen05 kernel (prefill_tcgen05.cuh), against which this independent second
// implementation is the tests' cross-check.
//
// Replaces the item walk of the reference's Attention::run
// (src/compiler/mul/attention.rs:85-153) together with the per-row key loop it
// calls (src/kernel/generic/flash_attention.rs:60-89): chunk row r of sequence b
// sits at absolute position base_b + r and attends keys 0..=base_b + r.
//
// A CTA owns 64 packed rows of one (sequence, KV head): packed row rho = r * G + g
// (g = query head inside the group, fastest), so the G query heads that share a KV
// head also share every K/V tile the CTA stages - the reference's "finish one head
// before moving to the next" locality, one level up.  K/V tiles of 64 keys are
// double-buffered in shared memory with cp.async.
#pragma once
#include "common.cuh"

namespace ellm {

constexpr int kPfWarps = 4;
constexpr int kPfThreads = kPfWarps * 32;
constexpr int kPfRows = kPfWarps * 16;   // packed rows per CTA
constexpr int kPfKeys = 64;              // keys per stage
constexpr int kPfStageBytes = kPfKeys * kRowBytes * 2;  // K + V
constexpr int kPfSmemBytes = 2 * kPfStageBytes;

struct PrefillParams {
    const __nv_bfloat16* q;     // [interval, max_batch, q_heads, 128]
    const __nv_bfloat16* k_cache;
    const __nv_bfloat16* v_cache;
    void* out;                  // bf16 or fp32, same indexing as q
    float* lse;                 // [interval, max_batch, q_heads] or nullptr
    const int32_t* positions;   // per-sequence chunk start, or nullptr
    long long position_index;
    long long key_begin, key_end;  // key window; [0, +inf) for the plain operator
    long long s0, s1, s2;
    int interval, batch, max_batch;
    int q_heads, kv_heads, group;
    int row_tiles;              // ceil(interval * group / 64)
    float scale_log2;
};

template <typename OutT>
__global__ void __launch_bounds__(kPfThreads, 2) prefill_warp_mma_kernel(const PrefillParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t smem_base = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // heaviest (latest) row tiles first: they have the longest key range
    const int tile = p.row_tiles - 1 - static_cast<int>(blockIdx.x);
    const int kvh = blockIdx.y, b = blockIdx.z;
    const long long base = p.positions ? static_cast<long long>(p.positions[b]) : p.position_index;
    const int total_rows = p.interval * p.group;
    const int rho_first = tile * kPfRows;
    const int rho_last = min(rho_first + kPfRows, total_rows) - 1;
    // keys this CTA needs: up to the causal limit of its last row, inside the window
    long long kend = base + rho_last / p.group + 1;
    if (kend > p.key_end) kend = p.key_end;
    const long long kbegin = p.key_begin;
    const int ntiles = kend > kbegin ? static_cast<int>((kend - kbegin + kPfKeys - 1) / kPfKeys) : 0;

    const __nv_bfloat16* kbase = p.k_cache + b * p.s0 + kvh * p.s1;
    const __nv_bfloat16* vbase = p.v_cache + b * p.s0 + kvh * p.s1;

    auto issue = [&](int it) {
        const long long kfirst = kbegin + static_cast<long long>(it) * kPfKeys;
        const uint32_t sK = smem_base + (it & 1) * kPfStageBytes;
        const uint32_t sV = sK + kPfKeys * kRowBytes;
        const int chunk = threadIdx.x & 15;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int row = (threadIdx.x >> 4) + 8 * i;
            const long long key = kfirst + row;
            const bool ok = key < kend;  // rows past the causal limit may hold anything: zero-fill
            const long long off = (ok ? key : 0) * p.s2 + chunk * 8;
            cp_async_16(sK + swz_off(row, chunk), kbase + off, ok ? 16 : 0);
            cp_async_16(sV + swz_off(row, chunk), vbase + off, ok ? 16 : 0);
        }
    };
    if (ntiles > 0) issue(0);
    cp_async_commit();

    // this thread's two packed rows
    const int r0 = lane >> 2;
    int rho[2] = {rho_first + warp * 16 + r0, rho_first + warp * 16 + r0 + 8};
    long long lim[2];   // last key (inclusive) each row may see
    long long qoff[2];  // element offset of the row in q / out
    bool valid[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        valid[r] = rho[r] < total_rows;
        const int pos = valid[r] ? rho[r] / p.group : 0, g = valid[r] ? rho[r] % p.group : 0;
        lim[r] = valid[r] ? base + pos : -1;
        qoff[r] = ((static_cast<long long>(pos) * p.max_batch + b) * p.q_heads + kvh * p.group + g) * kHeadDim;
    }
    uint32_t qf[8][4];
    {
        const int c0 = (lane & 3) * 2;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            qf[ks][0] = valid[0] ? *reinterpret_cast<const uint32_t*>(p.q + qoff[0] + ks * 16 + c0) : 0u;
            qf[ks][1] = valid[1] ? *reinterpret_cast<const uint32_t*>(p.q + qoff[1] + ks * 16 + c0) : 0u;
            qf[ks][2] = valid[0] ? *reinterpret_cast<const uint32_t*>(p.q + qoff[0] + ks * 16 + c0 + 8) : 0u;
            qf[ks][3] = valid[1] ? *reinterpret_cast<const uint32_t*>(p.q + qoff[1] + ks * 16 + c0 + 8) : 0u;
        }
    }
    // warp-uniform: last key any row of this warp may see
    long long warp_lim = base + min(rho_first + warp * 16 + 15, total_rows - 1) / p.group;
    if (rho_first + warp * 16 >= total_rows) warp_lim = -1;

    RowState st;
    st.m[0] = st.m[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.0f;
    float o[16][4];
#pragma unroll
    for (int nb = 0; nb < 16; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.0f;

    for (int it = 0; it < ntiles; ++it) {
        if (it + 1 < ntiles) issue(it + 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const long long kfirst = kbegin + static_cast<long long>(it) * kPfKeys;
        if (kfirst <= warp_lim) {
            const uint32_t sK = smem_base + (it & 1) * kPfStageBytes;
            float s[8][4];
            qk_step<8>(qf, sK, s, lane);
            const bool need_mask = kfirst + kPfKeys - 1 > base + (rho_first + warp * 16) / p.group ||
                                   kfirst + kPfKeys > kend;
            if (need_mask) {
                const long long kc = kfirst + (lane & 3) * 2;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const long long k0 = kc + 8 * j, k1 = k0 + 1;
                    s[j][0] = (k0 <= lim[0] && k0 < kend) ? s[j][0] * p.scale_log2 : -INFINITY;
                    s[j][1] = (k1 <= lim[0] && k1 < kend) ? s[j][1] * p.scale_log2 : -INFINITY;
                    s[j][2] = (k0 <= lim[1] && k0 < kend) ? s[j][2] * p.scale_log2 : -INFINITY;
                    s[j][3] = (k1 <= lim[1] && k1 < kend) ? s[j][3] * p.scale_log2 : -INFINITY;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    s[j][0] *= p.scale_log2; s[j][1] *= p.scale_log2;
                    s[j][2] *= p.scale_log2; s[j][3] *= p.scale_log2;
                }
            }
            softmax_pv_step<8>(s, st, o, sK + kPfKeys * kRowBytes, lane);
        }
        __syncthreads();  // stage (it & 1) is refilled by the next iteration's issue
    }
    cp_async_wait<0>();

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
    }
    OutT* out = reinterpret_cast<OutT*>(p.out);
    const int c0 = (lane & 3) * 2;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        if (!valid[r]) continue;
        const bool empty = st.l[r] == 0.0f;  // no key inside the window for this row
        const float inv = empty ? 0.0f : 1.0f / st.l[r];
#pragma unroll
        for (int nb = 0; nb < 16; ++nb) {
            const float x = o[nb][2 * r] * inv, y = o[nb][2 * r + 1] * inv;
            if constexpr (sizeof(OutT) == 4) {
                *reinterpret_cast<float2*>(reinterpret_cast<float*>(out) + qoff[r] + nb * 8 + c0) = make_float2(x, y);
            } else {
                *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(out) + qoff[r] + nb * 8 + c0) = pack_bf16(x, y);
            }
        }
        if (p.lse && (lane & 3) == 0)
            p.lse[qoff[r] / kHeadDim] = empty ? -INFINITY : (st.m[r] + log2f(st.l[r])) * kLn2;
    }
}

}  // namespace ellm
