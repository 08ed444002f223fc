// K2: split-KV decode attention, one new query row per sequence.  HBM-bound: every
// K and V row of every live sequence is read exactly once per call, whatever the
// number of query heads sharing it.
//
// Replaces, for position_interval == 1, the per-(sequence, query head) key loop of
// the reference kernel (src/kernel/x86_64/f16_512/flash_attention.rs:58-86, called
// per item from src/compiler/mul/attention.rs:117-153).
//
// Work decomposition.  A *segment* is one (sequence b, KV head, block of <=16 query
// heads of its group); its keys are cut into tiles of 64.  All tiles of all
// segments form one flat list which is split evenly over the resident CTAs with
// the reference's own partitioner rule (compiler::assign).  A CTA walks its
// contiguous tile range; each maximal run inside one segment is a *piece* and
// yields one fp32 partial (O, LSE) in the workspace, slot = cta + segment (unique
// because consecutive pieces advance the CTA index, the segment index or both).
// merge_partials.cuh then combines the pieces of each segment; it is launched as a
// programmatic dependent grid so that its set-up overlaps this kernel's tail.  (Merging
// inside this kernel - the CTA that finishes a segment's last piece combines them - was
// measured 12 us slower: the serial reads of the other pieces sit at the kernel's tail.)
// The append of the new token's K/V row rides along in this kernel.
//
// Inside a CTA the 4 warps are independent streams: warp w owns keys
// [16w, 16w+16) of every tile, copies them global->shared itself (cp.async, 16 B
// per lane, 512 B contiguous per instruction, XOR-swizzled rows), and keeps its
// own online-softmax state; the warps only meet at the end of a piece.  The
// products run on the warp-level tensor-core MMA with the warp's 16 KEYS as the M
// dimension and the group's query heads, 8 to a block, as N (decode_stage_t in
// common.cuh), so one K/V read serves the whole group and a group of 8 heads
// fills the MMA exactly.  NB = blocks of 8 heads per segment (1 for groups of up
// to 8 heads, else 2).
#pragma once
#include "common.cuh"

namespace ellm {

constexpr int kDecWarps = 4;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kDecTileKeys = 64;                  // keys per tile (16 per warp)
constexpr int kDecStages = 3;                     // cp.async ring depth per warp
constexpr int kDecWarpStageBytes = 16 * kRowBytes * 2;  // 16 K rows + 16 V rows = 8 KB
constexpr int kDecMaxBatch = 1024;                // prefix table held in shared memory
constexpr int kDecSmemBytes = kDecWarps * kDecStages * kDecWarpStageBytes + (2 * kDecMaxBatch + 1) * 4;

struct DecodeParams {
    const __nv_bfloat16* q;        // [max_batch, q_heads, 128] (chunk row 0)
    const __nv_bfloat16* k_cache;
    const __nv_bfloat16* v_cache;
    float* part_o;                 // [slots, 16, 128]
    float* part_lse;               // [slots, 16]
    const int32_t* positions;      // device int32[batch] or nullptr
    long long uniform_len;         // keys per sequence when positions == nullptr
    long long len_cap;             // no sequence is read past this many keys (cache rows / window end)
    long long key_begin;           // attend keys [key_begin, len) only (0 for a plain decode)
    long long s0, s1, s2;          // kv strides in elements (batch, head, position)
    int batch;
    int q_heads, kv_heads, group;  // group = q_heads / kv_heads
    int gtiles;                    // ceil(group / 16)
    float scale_log2;              // scale * log2(e)
    int num_ctas;
    // Fused KV append: when k_new is set, the new token's K/V row of sequence b (at position
    // positions[b], or uniform_len - 1) is read from k_new / v_new [max_batch, kv_heads, 128]
    // instead of the cache, and written into the cache by the CTA that streams it.
    const __nv_bfloat16* k_new = nullptr;
    const __nv_bfloat16* v_new = nullptr;
    __nv_bfloat16* k_cache_w = nullptr;
    __nv_bfloat16* v_cache_w = nullptr;
    // Early streaming (opt-in, see ellm_attn_set_option "decode_early_stream"): the tile table is
    // built and the first K/V stages are requested BEFORE the wait for the stream's previous kernel.
    // Only what that kernel cannot have written is touched early: the positions, and cache rows
    // below each sequence's newest row; the queries and the stages that hold a newest row wait.
    int early = 0;
};

// CTA index owning tile t under assign_range(total, n, .)
__device__ __forceinline__ long long cta_of_tile(long long total, long long n, long long t) {
    const long long q = total / n, r = total % n;
    if (t < (q + 1) * r) return t / (q + 1);
    return r + (t - (q + 1) * r) / q;
}

// Keys sequence b would attend without the cap: its new token sits at positions[b], so positions[b] + 1.
__device__ __forceinline__ long long dec_seq_len_raw(const DecodeParams& p, int b) {
    return p.positions ? static_cast<long long>(p.positions[b]) + 1 : p.uniform_len;
}

// Tiles of a sequence of `len` keys (all of its segments have the same count).
__device__ __forceinline__ int dec_tiles_of(const DecodeParams& p, long long len) {
    const long long n = len - p.key_begin;
    if (n <= 0) return 0;
    return static_cast<int>((n + kDecTileKeys - 1) / kDecTileKeys);
}

// prefix[b] = sum of tiles of sequences < b, for b in [0, batch]; lens[b] = keys sequence b would
// attend without the cap (the positions are read here once, by one thread per sequence, and never
// again: they may live in page-locked host memory).  All threads call.  The positions are fetched by as many threads as there are
// sequences (one global-memory latency, not one per sequence); the running sum over the
// per-sequence tile counts is then a short loop over shared memory.
__device__ inline void dec_build_prefix(const DecodeParams& p, int* prefix, int* lens) {
    for (int b = threadIdx.x; b < p.batch; b += blockDim.x) {
        const long long raw = dec_seq_len_raw(p, b);
        lens[b] = static_cast<int>(raw < 0 ? 0 : raw);
        prefix[b + 1] = dec_tiles_of(p, raw < p.len_cap ? raw : p.len_cap);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        prefix[0] = 0;
        for (int b = 0; b < p.batch; ++b) {
            acc += prefix[b + 1];
            prefix[b + 1] = acc;
        }
    }
    __syncthreads();
}

// Largest b with prefix[b] * segs_per_seq <= t  (t < total tiles), skipping empty
// sequences.
__device__ __forceinline__ int dec_find_seq(const int* prefix, int batch, long long segs_per_seq,
                                            long long t) {
    int lo = 0, hi = batch;  // invariant: prefix[lo]*S <= t < prefix[hi]*S
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (static_cast<long long>(prefix[mid]) * segs_per_seq <= t) lo = mid; else hi = mid;
    }
    return lo;
}

// Segment-aligned split.  The flat rule (assign_range over all tiles) gives every CTA the same
// number of tiles, but a CTA whose range crosses a segment boundary has two pieces: it drains its
// ring, combines and writes a partial, then starts again with an empty ring - about 3 us more than
// its neighbours, and the grid ends with its last CTA.  With many segments that is what the even
// split costs everywhere; with few (a step of one or a few sequences: every segment has many CTAs
// and the kernel is a few microseconds long) those few CTAs decide the step.  There the CTA
// boundaries are snapped to the segment boundaries instead: segment [P, P + T) of the flat tile
// list gets CTAs [snap(P), snap(P + T)), snap(x) = round(x * ctas / total), and splits its T tiles
// evenly over them, so every CTA has one piece.  The decision depends on the positions only and is
// taken identically by every CTA of the decode grid and of the merge grid.
// (only called where total <= 32 * ctas and ctas is a few hundred: 32-bit arithmetic, no 64-bit division)
__device__ __forceinline__ long long dec_snap(long long tile, long long total, long long ctas) {
    return static_cast<long long>((static_cast<unsigned>(tile) * static_cast<unsigned>(ctas) + static_cast<unsigned>(total) / 2u) /
                                  static_cast<unsigned>(total));
}
__device__ inline bool dec_split_is_aligned(const DecodeParams& p, const int* prefix, long long segs_per_seq, long long total) {
    // few segments, at least a tile per CTA, and short enough that a rounding of one CTA per segment
    // (at most 1/8 of a segment's share) costs less than the second pieces would
    if (static_cast<long long>(p.batch) * segs_per_seq * 8 > p.num_ctas || total < p.num_ctas || total > 32LL * p.num_ctas || p.num_ctas > 4096) return false;
    for (int b = 0; b < p.batch; ++b) {
        const long long tiles_b = prefix[b + 1] - prefix[b];
        if (tiles_b == 0) continue;
        const long long base = static_cast<long long>(prefix[b]) * segs_per_seq;
        for (long long j = 0; j < segs_per_seq; ++j)   // every segment needs a CTA of its own
            if (dec_snap(base + (j + 1) * tiles_b, total, p.num_ctas) == dec_snap(base + j * tiles_b, total, p.num_ctas)) return false;
    }
    return true;
}
// The tile range of CTA `cta` under the segment-aligned split; false when it has none.
__device__ inline bool dec_aligned_range(const DecodeParams& p, const int* prefix, long long segs_per_seq, long long total,
                                         long long cta, long long* t_begin, long long* t_end) {
    for (int b = 0; b < p.batch; ++b) {
        const long long tiles_b = prefix[b + 1] - prefix[b];
        if (tiles_b == 0) continue;
        const long long base = static_cast<long long>(prefix[b]) * segs_per_seq;
        if (cta >= dec_snap(base + segs_per_seq * tiles_b, total, p.num_ctas)) continue;   // a later sequence
        for (long long j = 0; j < segs_per_seq; ++j) {
            const long long first = base + j * tiles_b;
            const long long c0 = dec_snap(first, total, p.num_ctas), c1 = dec_snap(first + tiles_b, total, p.num_ctas);
            if (cta >= c0 && cta < c1) {
                long long lb, le;
                if (!assign_range(tiles_b, c1 - c0, cta - c0, &lb, &le)) return false;
                *t_begin = first + lb;
                *t_end = first + le;
                return true;
            }
        }
    }
    return false;
}

template <int NB>
__global__ void __launch_bounds__(kDecThreads, 2) decode_splitkv_kernel(const DecodeParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    int* prefix = reinterpret_cast<int*>(smem + kDecWarps * kDecStages * kDecWarpStageBytes);   // [kDecMaxBatch + 1]
    int* lens = prefix + kDecMaxBatch + 1;                                                        // [kDecMaxBatch]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t warp_smem = smem_u32(smem) + warp * kDecStages * kDecWarpStageBytes;
    ChainTrace ct(2);

    // Under a programmatic dependent launch of this grid, wait here for the kernel before it (it
    // wrote the positions, the queries and the newest cache row); a no-op for an ordinary launch.
    // Only then let the dependent grid (the merge) be set up: whatever it does before its own wait
    // - it rebuilds the tile table from the positions - then sees everything this grid sees.
    // With early streaming the wait comes later, after the first stages have been requested.
    bool waited = p.early == 0;
    if (waited) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        ct.waited();
    }
    dec_build_prefix(p, prefix, lens);
    const long long segs_per_seq = static_cast<long long>(p.kv_heads) * p.gtiles;
    const long long total = static_cast<long long>(prefix[p.batch]) * segs_per_seq;
    long long t_begin = 0, t_end = 0;
    const bool has_tiles = dec_split_is_aligned(p, prefix, segs_per_seq, total)
                               ? dec_aligned_range(p, prefix, segs_per_seq, total, blockIdx.x, &t_begin, &t_end)
                               : assign_range(total, p.num_ctas, blockIdx.x, &t_begin, &t_end);
    if (!has_tiles) {
        if (!waited) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        return;
    }

    long long t = t_begin;
    while (t < t_end) {
        // ---- locate the piece: segment of tile t and how far it runs ----
        const int b = dec_find_seq(prefix, p.batch, segs_per_seq, t);
        const int tiles_b = prefix[b + 1] - prefix[b];
        const long long seq_base = static_cast<long long>(prefix[b]) * segs_per_seq;
        const int seg_in_seq = static_cast<int>((t - seq_base) / tiles_b);
        const int tile0 = static_cast<int>((t - seq_base) % tiles_b);
        const long long seg_end = seq_base + static_cast<long long>(seg_in_seq + 1) * tiles_b;
        const long long piece_end = seg_end < t_end ? seg_end : t_end;
        const int ntiles = static_cast<int>(piece_end - t);
        const int kvh = seg_in_seq / p.gtiles, gt = seg_in_seq % p.gtiles;
        const long long segment = static_cast<long long>(b) * segs_per_seq + seg_in_seq;
        const long long len_raw = lens[b];
        const long long len = len_raw < p.len_cap ? len_raw : p.len_cap;
        const int rows_valid = min(16, p.group - gt * 16);
        const long long key0 = p.key_begin + static_cast<long long>(tile0) * kDecTileKeys + warp * 16;
        const __nv_bfloat16* kbase = p.k_cache + b * p.s0 + kvh * p.s1;
        const __nv_bfloat16* vbase = p.v_cache + b * p.s0 + kvh * p.s1;
        // fused append: position of the new token's row and where its K/V come from
        // the row being appended is the sequence's last key, unless its position lies past the
        // cache (then len was capped and nothing is read or written there)
        long long new_pos = -1;
        if (p.k_new && len_raw == len) new_pos = len - 1;
        const __nv_bfloat16* knew = p.k_new ? p.k_new + (static_cast<long long>(b) * p.kv_heads + kvh) * kHeadDim : nullptr;
        const __nv_bfloat16* vnew = p.k_new ? p.v_new + (static_cast<long long>(b) * p.kv_heads + kvh) * kHeadDim : nullptr;

        // ---- cp.async ring: lane copies chunk (lane&15) of rows (lane>>4) + 2*i ----
        auto issue = [&](int it) {
            const long long kfirst = key0 + static_cast<long long>(it) * kDecTileKeys;
            const uint32_t sK = warp_smem + (it % kDecStages) * kDecWarpStageBytes;
            const uint32_t sV = sK + 16 * kRowBytes;
            const int chunk = lane & 15;
            // only the 16 keys that hold the segment's last key can contain the row being appended
            const bool has_new = new_pos >= kfirst && new_pos < kfirst + 16;
            if (!has_new) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int row = (lane >> 4) + 2 * i;
                    const long long key = kfirst + row;
                    const bool ok = key < len;
                    const long long off = (ok ? key : 0) * p.s2 + chunk * 8;
                    cp_async_16(sK + swz_off(row, chunk), kbase + off, ok ? 16 : 0);
                    cp_async_16(sV + swz_off(row, chunk), vbase + off, ok ? 16 : 0);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int row = (lane >> 4) + 2 * i;
                    const long long key = kfirst + row;
                    const bool ok = key < len;
                    const long long off = (ok ? key : 0) * p.s2 + chunk * 8;
                    if (key == new_pos) {   // stream the new row from k_new / v_new ...
                        cp_async_16(sK + swz_off(row, chunk), knew + chunk * 8, 16);
                        cp_async_16(sV + swz_off(row, chunk), vnew + chunk * 8, 16);
                        if (gt == 0) {      // ... and put it into the cache (once per KV head)
                            const long long woff = b * p.s0 + kvh * p.s1 + key * p.s2 + chunk * 8;
                            *reinterpret_cast<uint4*>(p.k_cache_w + woff) = *reinterpret_cast<const uint4*>(knew + chunk * 8);
                            *reinterpret_cast<uint4*>(p.v_cache_w + woff) = *reinterpret_cast<const uint4*>(vnew + chunk * 8);
                        }
                    } else {
                        cp_async_16(sK + swz_off(row, chunk), kbase + off, ok ? 16 : 0);
                        cp_async_16(sV + swz_off(row, chunk), vbase + off, ok ? 16 : 0);
                    }
                }
            }
        };
        int s_first = 0;
        if (!waited) {
            // the CTA's first piece: request ahead of the wait whatever cannot hold a row the
            // previous kernel writes (a sequence's newest row, at len - 1), stage by stage in order
            // (the stages the prologue below would request; filling the third ring slot as well was
            // measured 1 us slower per step, early or not: the loop's extra test changes its code)
#pragma unroll
            for (int s = 0; s < kDecStages - 1; ++s) {
                const long long kfirst = key0 + static_cast<long long>(s) * kDecTileKeys;
                const bool safe = s < ntiles && (len - 1 < kfirst || len - 1 >= kfirst + 16);
                if (s == s_first && safe) {
                    issue(s);
                    cp_async_commit();
                    ++s_first;
                }
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            waited = true;
            ct.waited();
        }
        // every stage is its own group and the groups are committed in stage order, so "all but the
        // last kDecStages - 1 groups have landed" below always covers the stage an iteration needs
#pragma unroll
        for (int s = 0; s < kDecStages - 1; ++s) {
            if (s >= s_first) {
                if (s < ntiles) issue(s);
                cp_async_commit();
            }
        }

        // ---- Q as B fragments: head nb*8 + lane/4 of the segment, dims ks*16 + (lane%4)*2 (+1), +8 ----
        uint32_t qb[NB][8][2];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const int head = nb * 8 + (lane >> 2);
            const bool hv = head < rows_valid;
            const __nv_bfloat16* qrow =
                p.q + (static_cast<long long>(b) * p.q_heads + kvh * p.group + gt * 16 + (hv ? head : 0)) * kHeadDim + (lane & 3) * 2;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                qb[nb][ks][0] = hv ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16) : 0u;
                qb[nb][ks][1] = hv ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8) : 0u;
            }
        }

        float hm[NB][2], hl[NB][2], oT[NB][8][4];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            hm[nb][0] = hm[nb][1] = -INFINITY;
            hl[nb][0] = hl[nb][1] = 0.0f;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) oT[nb][mt][0] = oT[nb][mt][1] = oT[nb][mt][2] = oT[nb][mt][3] = 0.0f;
        }

        for (int it = 0; it < ntiles; ++it) {
            if (it + kDecStages - 1 < ntiles) issue(it + kDecStages - 1);
            cp_async_commit();
            cp_async_wait<kDecStages - 1>();
            __syncwarp();
            const long long kfirst = key0 + static_cast<long long>(it) * kDecTileKeys;
            if (kfirst < len) {  // warp-uniform: this warp's 16 keys are not all past the end
                const uint32_t sK = warp_smem + (it % kDecStages) * kDecWarpStageBytes;
                decode_stage_t<NB>(qb, sK, sK + 16 * kRowBytes, kfirst, len, p.scale_log2, hm, hl, oT, lane);
            }
            __syncwarp();  // all lanes done with this stage before it is refilled
        }
        cp_async_wait<0>();
        ct.mid();   // (trace) the CTA's first piece has been streamed

        // ---- end of piece: combine the 4 warps through shared memory ----
        // a head's sum is spread over the 8 lanes that share lane%4 (their keys differ)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                hl[nb][h] += __shfl_xor_sync(0xffffffffu, hl[nb][h], 4);
                hl[nb][h] += __shfl_xor_sync(0xffffffffu, hl[nb][h], 8);
                hl[nb][h] += __shfl_xor_sync(0xffffffffu, hl[nb][h], 16);
            }
        __syncthreads();  // every warp has drained its ring; smem is free
        float* so = reinterpret_cast<float*>(smem);             // [warps][16 heads][128]
        float* sm = so + kDecWarps * 16 * kHeadDim;             // [warps][16]
        float* sl = sm + kDecWarps * 16;                        // [warps][16]
        {
            float* wo = so + warp * 16 * kHeadDim;
            const int d0 = lane >> 2, h0 = (lane & 3) * 2;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
                for (int mt = 0; mt < 8; ++mt) {
                    float* col = wo + (nb * 8 + h0) * kHeadDim + mt * 16 + d0;
                    col[0] = oT[nb][mt][0];
                    col[kHeadDim] = oT[nb][mt][1];
                    col[8] = oT[nb][mt][2];
                    col[kHeadDim + 8] = oT[nb][mt][3];
                }
                if ((lane >> 2) == 0) {
                    sm[warp * 16 + nb * 8 + h0] = hm[nb][0];
                    sm[warp * 16 + nb * 8 + h0 + 1] = hm[nb][1];
                    sl[warp * 16 + nb * 8 + h0] = hl[nb][0];
                    sl[warp * 16 + nb * 8 + h0 + 1] = hl[nb][1];
                }
            }
        }
        __syncthreads();
        {
            const long long slot = static_cast<long long>(blockIdx.x) + segment;
            float* po = p.part_o + slot * 16 * kHeadDim;
            for (int idx = threadIdx.x; idx < rows_valid * (kHeadDim / 4); idx += kDecThreads) {
                const int r = idx / (kHeadDim / 4), c4 = (idx % (kHeadDim / 4)) * 4;
                float mmax = -INFINITY;
#pragma unroll
                for (int w = 0; w < kDecWarps; ++w) mmax = fmaxf(mmax, sm[w * 16 + r]);
                float lsum = 0.0f;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int w = 0; w < kDecWarps; ++w) {
                    const float mw = sm[w * 16 + r];
                    const float a = (mw == -INFINITY) ? 0.0f : fast_exp2(mw - mmax);
                    lsum += a * sl[w * 16 + r];
                    const float4 x = *reinterpret_cast<const float4*>(so + (w * 16 + r) * kHeadDim + c4);
                    acc.x += a * x.x; acc.y += a * x.y; acc.z += a * x.z; acc.w += a * x.w;
                }
                const float inv = 1.0f / lsum;
                acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
                *reinterpret_cast<float4*>(po + r * kHeadDim + c4) = acc;
                if (c4 == 0) p.part_lse[slot * 16 + r] = (mmax + log2f(lsum)) * kLn2;
            }
        }
        __syncthreads();  // smem is reused by the next piece's ring
        t = piece_end;
    }
}

}  // namespace ellm
