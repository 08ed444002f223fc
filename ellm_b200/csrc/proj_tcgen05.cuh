// K6: the projections either side of attention on the Blackwell tensor cores.
//
//   C[M x N] = A[M x K] . W_nt[N x K]^T        bf16 operands, fp32 accumulation in tensor memory
//
// with one of two epilogues:
//   * plain / residual: C = (residual +) A.W^T, rounded once to bf16 - the reference's MatMul
//     and MatMulAdd (src/compiler/mul/matmul_add.rs:128-232: C = residual, C += A x B);
//   * fused QKV: the three projections of one attention block as one launch over the column
//     tiles of Wq, Wk, Wv, and on each finished 128-wide head the reference's finalize step
//     (src/compiler/mul/matmul3.rs:230-262 -> rms_norm + complex_mul on Q and K heads,
//     src/kernel/x86_64/f16_512/matmul_rms_complex.rs:76-96), the rotation row taken at the
//     token's position, K and V written straight into the static cache
//     (output_to_kv, src/compiler/zip_map/complex_zip.rs:92-98).  A column tile belongs to
//     exactly one of the three weights, like the reference's task list (matmul3.rs:264-287).
//
// Persistent kernel, one CTA per SM, tiles of 128 rows x 256 columns taken round-robin with
// the column tile fastest (the CTAs running together share a few A row blocks and all of W
// through L2).  Warp roles:
//   warp 0     TMA producer (one lane): A and W blocks of 64 k-elements through a 4-slot ring
//   warp 1     MMA issuer (one lane), owner of the 512 tensor-memory columns = two accumulators
//   warps 2-9  epilogue: thread = one row of the tile and one half of its columns (one head of
//              the two); the accumulator of tile i is drained while the MMAs of tile i+1 fill
//              the other one.  Eight warps because an epilogue is a chain of latencies (tensor-
//              memory load, rotation rows from L2, conversions): two warps per scheduler overlap them
// Every wait is bounded; on expiry a status word is set and all roles leave (see
// prefill_tcgen05.cuh, whose barrier, TMA and descriptor helpers this file uses).
#pragma once
#include "prefill_tcgen05.cuh"

namespace ellm {

constexpr int kPjBM = 128;         // rows per tile = tensor-memory lanes
constexpr int kPjBN = 256;         // columns per tile = two heads
constexpr int kPjBK = 64;          // k-elements per ring slot: one 128-byte swizzled row
constexpr int kPjABytes = kPjBM * 128;                 // 16 KB
// One CTA per tile: 4 ring slots of A (16 KB) + W (256 rows, 32 KB).  Two CTAs per 256 x 256 tile
// (cta_group::2): 6 slots of A (this CTA's 128 rows) + half of W (this CTA's 128 of the 256 columns).
template <bool kPair> struct PjRing {
    static constexpr int kStages = kPair ? 6 : 4;
    static constexpr int kBBytes = kPair ? 128 * 128 : kPjBN * 128;
    static constexpr int kStageBytes = kPjABytes + kBBytes;
};
constexpr int kPjSmemBar = PjRing<false>::kStages * PjRing<false>::kStageBytes;   // 192 KB either way
static_assert(PjRing<true>::kStages * PjRing<true>::kStageBytes == kPjSmemBar, "both rings fill the same space");
constexpr int kPjEpiWarps = 8;                          // two per tensor-memory lane quarter
constexpr int kPjRopePitch = 64 + 16;                   // a staged piece of a rotation row (16 floats) + pad against bank conflicts
constexpr int kPjStageWarpBytes = 32 * kPjRopePitch;    // per epilogue warp
constexpr int kPjSmemStage = kPjSmemBar + 256;
constexpr int kPjSmemBytes = kPjSmemStage + kPjEpiWarps * kPjStageWarpBytes + 1024;  // + slack to align the base to 1024
static_assert(kPjSmemBytes <= 232448, "shared memory budget");
constexpr int kPjThreads = (2 + kPjEpiWarps) * 32;

enum { kPjWaitFull = 11, kPjWaitEmpty = 12, kPjWaitAccFull = 13, kPjWaitAccEmpty = 14 };
enum { kPjPlain = 0, kPjQkv = 1 };

struct ProjParams {
    int mode;                 // kPjPlain or kPjQkv
    int m_rows;               // rows of A that exist: chunk rows x max_batch
    int k_blocks;             // K / 64
    int tiles_m;              // row tiles: of 128 rows, or of 256 rows for CTA pairs
    int tiles_n;              // all column tiles; in kPjQkv = tiles_q + 2 * tiles_kv
    int tiles_q, tiles_kv;    // kPjQkv: column tiles of Wq and of Wk (= of Wv)
    int* status;
    unsigned long long wait_timeout_ns;
    int debug_skip_load;      // test hook: ring item of CTA 0 the producer never loads (its barrier stays unsignalled); -1 = none
    int batch, max_batch;     // rows are (chunk row r, sequence b) = r * max_batch + b; rows with b >= batch are skipped
    // ---- kPjPlain
    __nv_bfloat16* c;
    const __nv_bfloat16* residual;   // or nullptr
    long long ldc, ldr;       // elements
    int n_cols;
    // ---- kPjQkv
    __nv_bfloat16* q_out;     // [rows, q_heads, 128]
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    const float* q_weight;    // [128] or nullptr
    const float* k_weight;
    const float* rope;        // [rope_rows, 128] interleaved (cos, sin)
    const int32_t* positions; // per-sequence chunk start or nullptr
    long long position_index;
    long long s0, s1, s2;
    long long max_seq, rope_rows;
    int q_heads, kv_heads;
    float eps;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

// bf16 x bf16 -> fp32, M = m (128 for one CTA, 256 over a CTA pair), N = n, both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc_mn(uint32_t m, uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---- CTA pairs: two CTAs of a cluster share one 256 x 256 tile; CTA 0 issues the MMAs for both
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the shared::cluster address of `addr` (a shared-memory address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into this CTA's shared memory whose completion is counted on a barrier that may live in the pair's other CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrival on a barrier (of either CTA of the pair) once every MMA issued so far has completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// One head (128 accumulator columns starting at `taddr`) of the warp's 32 rows: rounded to bf16
// like the stored projection the unfused path would read back, then norm, rotation and the
// store.  kind 0 = Q, 1 = K, 2 = V.  A thread owns a row (its tensor-memory lane).  Rotation rows
// are 512 bytes apart, so the warp fetches them 8 rows per instruction (16 channels at a time,
// two pieces ahead of their use, held in registers) and passes them through a small per-warp
// shared-memory stage from which every thread reads its own row.
__device__ __forceinline__ void proj_head_epilogue(const ProjParams& p, uint32_t taddr, int kind, int head, long long m,
                                                   int b, long long pos, bool live, unsigned char* stage, int lane) {
    __syncwarp();
    bool store = live;
    if (kind != 0 && (pos < 0 || pos >= p.max_seq)) store = false;
    if (pos < 0 || pos >= p.rope_rows) store = false;   // no rotation row: leave Q and the token's whole cache line (K and V) untouched
    __nv_bfloat16* dst = kind == 0 ? p.q_out + (m * p.q_heads + head) * kHeadDim
                                   : (kind == 1 ? p.k_cache : p.v_cache) + b * p.s0 + head * p.s1 + pos * p.s2;
    if (kind == 2) {   // V: the projected row as it is
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float v[32];
            tmem_ld32(taddr + c * 32, v);
            tmem_wait_ld();
            if (store) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) =
                        make_uint4(pack_bf16(v[i * 8 + 0], v[i * 8 + 1]), pack_bf16(v[i * 8 + 2], v[i * 8 + 3]),
                                   pack_bf16(v[i * 8 + 4], v[i * 8 + 5]), pack_bf16(v[i * 8 + 6], v[i * 8 + 7]));
            }
        }
        return;
    }
    // piece c of the rotation rows: lane fetches 16 bytes of row 8*i + lane/4, i = 0..3
    const unsigned long long rope_bits = reinterpret_cast<unsigned long long>(p.rope + (store ? pos : 0) * kHeadDim);
    unsigned long long src_row[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) src_row[i] = __shfl_sync(0xffffffffu, rope_bits, i * 8 + (lane >> 2));
    auto fetch = [&](float4 (&r)[4], int c) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            r[i] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src_row[i]) + c * 16 + (lane & 3) * 4);
    };
    float4 ahead[2][4];
    fetch(ahead[0], 0);
    fetch(ahead[1], 1);
    // pass 1: the sum of squares of the rounded row
    float ss0 = 0.0f, ss1 = 0.0f, ss2 = 0.0f, ss3 = 0.0f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        float v[32];
        tmem_ld32(taddr + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float a0 = bf16_round(v[4 * i]), a1 = bf16_round(v[4 * i + 1]);
            const float a2 = bf16_round(v[4 * i + 2]), a3 = bf16_round(v[4 * i + 3]);
            ss0 = fmaf(a0, a0, ss0);
            ss1 = fmaf(a1, a1, ss1);
            ss2 = fmaf(a2, a2, ss2);
            ss3 = fmaf(a3, a3, ss3);
        }
    }
    const float ss = (ss0 + ss1) + (ss2 + ss3);
    const float rrms = 1.0f / (sqrtf(ss / static_cast<float>(kHeadDim)) + p.eps);
    const float* wgt = kind == 0 ? p.q_weight : p.k_weight;
    // pass 2: 16 channels = 8 rotation pairs at a time
#pragma unroll
    for (int c = 0; c < 8; ++c) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            *reinterpret_cast<float4*>(stage + (i * 8 + (lane >> 2)) * kPjRopePitch + (lane & 3) * 16) = ahead[c & 1][i];
        __syncwarp();
        if (c + 2 < 8) fetch(ahead[c & 1], c + 2);
        float v[16];
        tmem_ld16(taddr + c * 16, v);
        tmem_wait_ld();
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {   // channels 16c + 4j .. +3
            const float4 r = *reinterpret_cast<const float4*>(stage + lane * kPjRopePitch + j * 16);   // cos0 sin0 cos1 sin1
            float4 wv = make_float4(1.f, 1.f, 1.f, 1.f);
            if (wgt) wv = *reinterpret_cast<const float4*>(wgt + c * 16 + j * 4);
            const float y0 = bf16_round(v[4 * j]) * rrms * wv.x, y1 = bf16_round(v[4 * j + 1]) * rrms * wv.y;
            const float y2 = bf16_round(v[4 * j + 2]) * rrms * wv.z, y3 = bf16_round(v[4 * j + 3]) * rrms * wv.w;
            o[j * 2] = pack_bf16(y0 * r.x - y1 * r.y, y0 * r.y + y1 * r.x);
            o[j * 2 + 1] = pack_bf16(y2 * r.z - y3 * r.w, y2 * r.w + y3 * r.z);
        }
        __syncwarp();   // the stage may be overwritten
        if (store) {
            *reinterpret_cast<uint4*>(dst + c * 16) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(dst + c * 16 + 8) = make_uint4(o[4], o[5], o[6], o[7]);
        }
    }
}

template <bool kPair>
__global__ void __launch_bounds__(kPjThreads, 1)
proj_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w0,
                    const __grid_constant__ CUtensorMap map_w1, const __grid_constant__ CUtensorMap map_w2,
                    const ProjParams p) {
    constexpr int kStages = PjRing<kPair>::kStages, kStageBytes = PjRing<kPair>::kStageBytes;
    constexpr int kTileRows = kPair ? 2 * kPjBM : kPjBM;   // rows of a tile over the CTA(s) that share it
    extern __shared__ unsigned char smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the kernel that follows (attention, launched as a programmatic dependent) may be set up now
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // pair mode: `rank` is this CTA's place in its pair, `unit` the pair's number; CTA 0 of a pair leads
    const int rank = kPair ? static_cast<int>(cluster_ctarank()) : 0;
    const int unit = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int units = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

    const uint32_t bar0 = smem_base + kPjSmemBar;
    auto bar_full = [&](int s) { return bar0 + 8u * s; };                        // used in the leader only
    auto bar_empty = [&](int s) { return bar0 + 8u * (kStages + s); };
    auto bar_acc_full = [&](int a) { return bar0 + 8u * (2 * kStages + a); };
    auto bar_acc_empty = [&](int a) { return bar0 + 8u * (2 * kStages + 2 + a); };   // used in the leader only
    constexpr int kNumBars = 2 * kStages + 4;
    static_assert(8 * kNumBars + 16 <= 256, "barrier region too small");
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kPjSmemBar + 8 * kNumBars);
    volatile int* abort_word = reinterpret_cast<volatile int*>(smem + kPjSmemBar + 8 * kNumBars + 8);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_acc_full(a), 1);
            mbar_init(bar_acc_empty(a), kPjEpiWarps * (kPair ? 2 : 1));   // one arrival per epilogue warp (of both CTAs)
        }
        *abort_word = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // in pair mode the same warp of both CTAs allocates together
        if constexpr (kPair) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (kPair) cluster_sync_all();   // the other CTA's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int total_tiles = p.tiles_m * p.tiles_n;

    if (warp == 0) {
        // =============================== TMA producer ===============================
        if (lane == 0) {
            bool ok = true;
            int item = 0;
            for (int tile = unit; tile < total_tiles && ok; tile += units) {
                const int tm = tile / p.tiles_n, tn = tile % p.tiles_n;
                const CUtensorMap* map_w = &map_w0;
                int n0 = tn * kPjBN;
                if (p.mode == kPjQkv && tn >= p.tiles_q) {
                    const bool is_k = tn < p.tiles_q + p.tiles_kv;
                    map_w = is_k ? &map_w1 : &map_w2;
                    n0 = (tn - p.tiles_q - (is_k ? 0 : p.tiles_kv)) * kPjBN;
                }
                for (int kb = 0; kb < p.k_blocks; ++kb, ++item) {
                    const int slot = item % kStages, round = item / kStages;
                    ok = mbar_wait(bar_empty(slot), (round & 1) ^ 1, abort_word, p.status, kPjWaitEmpty, p.wait_timeout_ns);
                    if (!ok) break;
                    if (item == p.debug_skip_load && blockIdx.x == 0) continue;   // test hook: this block never arrives
                    const uint32_t dst = smem_base + slot * kStageBytes;
                    if constexpr (kPair) {
                        // both CTAs' loads are counted on the leader's barrier: its own 32 KB and the other CTA's
                        if (rank == 0) mbar_arrive_expect_tx(bar_full(slot), 2 * kStageBytes);
                        const uint32_t full = mapa_shared(bar_full(slot), 0);
                        tma_load_2d_pair(dst, &map_a, full, kb * kPjBK, tm * kTileRows + rank * kPjBM);
                        tma_load_2d_pair(dst + kPjABytes, map_w, full, kb * kPjBK, n0 + rank * (kPjBN / 2));
                    } else {
                        mbar_arrive_expect_tx(bar_full(slot), kStageBytes);
                        tma_load_2d(dst, &map_a, bar_full(slot), kb * kPjBK, tm * kPjBM);
                        tma_load_2d(dst + kPjABytes, map_w, bar_full(slot), kb * kPjBK, n0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // =============================== MMA issuer ===============================
        if (lane == 0 && rank == 0) {
            bool ok = true;
            constexpr uint32_t idesc = umma_idesc_mn(kTileRows, kPjBN);
            int item = 0, local = 0;
            for (int tile = unit; tile < total_tiles && ok; tile += units, ++local) {
                const int acc = local & 1;
                ok = mbar_wait(bar_acc_empty(acc), ((local >> 1) & 1) ^ 1, abort_word, p.status, kPjWaitAccEmpty, p.wait_timeout_ns);
                if (!ok) break;
                tc_fence_after();
                for (int kb = 0; kb < p.k_blocks; ++kb, ++item) {
                    const int slot = item % kStages, round = item / kStages;
                    ok = mbar_wait(bar_full(slot), round & 1, abort_word, p.status, kPjWaitFull, p.wait_timeout_ns);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_base + slot * kStageBytes, b_addr = a_addr + kPjABytes;
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        if constexpr (kPair)   // operands at the same offsets in both CTAs: A rows 128 + 128, W columns 128 + 128
                            umma_bf16_pair(tmem + acc * kPjBN, umma_desc(a_addr + ks * 32, 0, 1024),
                                           umma_desc(b_addr + ks * 32, 0, 1024), idesc, (kb | ks) != 0);
                        else
                            umma_bf16(tmem + acc * kPjBN, umma_desc(a_addr + ks * 32, 0, 1024), umma_desc(b_addr + ks * 32, 0, 1024),
                                      idesc, (kb | ks) != 0);
                    }
                    if constexpr (kPair) {   // the slot is free in both CTAs
                        umma_commit_pair(bar_empty(slot));
                        umma_commit_pair(mapa_shared(bar_empty(slot), 1));
                    } else {
                        umma_commit(bar_empty(slot));
                    }
                }
                if (ok) {
                    if constexpr (kPair) {
                        umma_commit_pair(bar_acc_full(acc));
                        umma_commit_pair(mapa_shared(bar_acc_full(acc), 1));
                    } else {
                        umma_commit(bar_acc_full(acc));
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // =============================== epilogue ===============================
        const int quarter = warp & 3;   // the tensor-memory lanes a warp may touch: 32 * (warp % 4) ...
        const int part = (warp - 2) >> 2;   // which half of the tile's columns (which of its two heads)
        const int row = quarter * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        bool ok = true;
        int local = 0;
        for (int tile = unit; tile < total_tiles && ok; tile += units, ++local) {
            const int acc = local & 1;
            const int tm = tile / p.tiles_n, tn = tile % p.tiles_n;
            ok = lane == 0 ? mbar_wait(bar_acc_full(acc), (local >> 1) & 1, abort_word, p.status, kPjWaitAccFull, p.wait_timeout_ns) : true;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t tacc = tmem + lane_base + acc * kPjBN;
            const long long m = static_cast<long long>(tm) * kTileRows + rank * kPjBM + row;
            const int b = static_cast<int>(m % p.max_batch);
            const bool live = m < p.m_rows && b < p.batch;
            if (p.mode == kPjPlain) {
                const int n0 = tn * kPjBN + part * 128;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    if (n0 + c * 32 >= p.n_cols) break;   // warp-uniform
                    float v[32];
                    tmem_ld32(tacc + part * 128 + c * 32, v);
                    uint4 rv[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {   // residual pieces requested before the accumulator is needed
                        rv[i] = make_uint4(0u, 0u, 0u, 0u);
                        const int n = n0 + c * 32 + i * 8;
                        if (live && p.residual && n < p.n_cols) rv[i] = *reinterpret_cast<const uint4*>(p.residual + m * p.ldr + n);
                    }
                    tmem_wait_ld();
                    if (live) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int n = n0 + c * 32 + i * 8;
                            const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv[i]);
                            uint4 o;
                            o.x = pack_bf16(v[i * 8 + 0] + __low2float(r2[0]), v[i * 8 + 1] + __high2float(r2[0]));
                            o.y = pack_bf16(v[i * 8 + 2] + __low2float(r2[1]), v[i * 8 + 3] + __high2float(r2[1]));
                            o.z = pack_bf16(v[i * 8 + 4] + __low2float(r2[2]), v[i * 8 + 5] + __high2float(r2[2]));
                            o.w = pack_bf16(v[i * 8 + 6] + __low2float(r2[3]), v[i * 8 + 7] + __high2float(r2[3]));
                            if (n < p.n_cols) *reinterpret_cast<uint4*>(p.c + m * p.ldc + n) = o;
                        }
                    }
                }
            } else {
                int kind = 0, head0 = tn * 2, heads = p.q_heads;
                if (tn >= p.tiles_q + p.tiles_kv) {
                    kind = 2;
                    head0 = (tn - p.tiles_q - p.tiles_kv) * 2;
                    heads = p.kv_heads;
                } else if (tn >= p.tiles_q) {
                    kind = 1;
                    head0 = (tn - p.tiles_q) * 2;
                    heads = p.kv_heads;
                }
                const long long r = m / p.max_batch;
                const long long pos = (p.positions ? static_cast<long long>(p.positions[live ? b : 0]) : p.position_index) + r;
                if (head0 + part < heads)
                    proj_head_epilogue(p, tacc + part * 128, kind, head0 + part, m, b, pos, live,
                                       smem + kPjSmemStage + (warp - 2) * kPjStageWarpBytes, lane);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if constexpr (kPair) mbar_arrive_cluster(mapa_shared(bar_acc_empty(acc), 0));
                else mbar_arrive(bar_acc_empty(acc));
            }
        }
    }

    // teardown: every role gets here (all waits are bounded)
    tc_fence_before();
    __syncthreads();
    if (*abort_word) {
        // a wait ran out: TMA copies may still be in flight towards this CTA's shared memory
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    // neither CTA of a pair goes away while the other may still signal its barriers or read its operands
    if constexpr (kPair) cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        if constexpr (kPair) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
    }
}

// ---------------------------------------------------------------- host side
struct ProjPlan {
    bool ready = false;
    char why[160] = "";
    void* encode = nullptr;
    int sm_count = 0;
    unsigned long long wait_timeout_ns = 2000000000ull;
    int debug_skip_load = -1;
    int pairing = -1;   // CTA pairs per 256 x 256 tile: -1 = when the problem has enough tiles, 0 = never, 1 = whenever possible
};

inline void proj_plan_init(ProjPlan& plan, int sm_count) {
    plan.ready = false;
    plan.sm_count = sm_count;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn ||
        qres != cudaDriverEntryPointSuccess) {
        cudaGetLastError();
        snprintf(plan.why, sizeof(plan.why), "driver does not export cuTensorMapEncodeTiled");
        return;
    }
    if (cudaFuncSetAttribute(proj_tcgen05_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPjSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(proj_tcgen05_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPjSmemBytes) != cudaSuccess) {
        snprintf(plan.why, sizeof(plan.why), "cannot reserve %d bytes of shared memory: %s", kPjSmemBytes,
                 cudaGetErrorString(cudaGetLastError()));
        return;
    }
    plan.encode = fn;
    plan.ready = true;
}

// A row-major bf16 matrix [rows x cols] with `ld` elements between rows, as boxes of 64 columns x box_rows rows.
inline bool proj_encode_2d(const ProjPlan& plan, CUtensorMap* map, const void* base, size_t rows, size_t cols, size_t ld,
                           unsigned box_rows) {
    EncodeTiledFn encode = reinterpret_cast<EncodeTiledFn>(plan.encode);
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t es[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace ellm
