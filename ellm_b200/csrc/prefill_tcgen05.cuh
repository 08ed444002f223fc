// K1 (fast form): causal grouped-query flash-attention prefill on the Blackwell
// tensor cores: tcgen05.mma with accumulators in tensor memory, operands staged in
// shared memory by TMA (no cluster, no multicast), online softmax in fp32.
//
// Replaces, for chunks of many rows, the item walk of the reference's
// Attention::run (src/compiler/mul/attention.rs:85-153) and the per-row key loop
// it calls (src/kernel/generic/flash_attention.rs:60-89): chunk row r of sequence
// b is the token at position base + r and attends keys 0..=base + r.
//
// A work item is 256 packed rows of one (sequence, KV head): packed row rho = r*G + g
// (g = query head inside its group, fastest), split in two tiles of 128 rows, so
// the G query heads of a group share every K/V tile - the reference's "one KV
// head at a time" locality.  One CTA per SM walks the list of items (heaviest
// first, the next untaken one from a device counter).  Warp roles:
//   warps 0-3  softmax / correction / epilogue of tile 0 (thread = one row)
//   warps 4-7  the same for tile 1
//   warp  8    TMA producer (one lane): Q tiles once, then K_j, V_j through a ring
//   warp  9    MMA issuer (one lane) and owner of the tensor-memory allocation
// Per 128-key tile j and row tile t:  S_t = Q_t K_j^T (tensor memory) -> softmax
// threads read S_t half a row at a time, write P_t (bf16) back into the first 64
// columns of S_t (the first half's P before the second half's scores are fetched)
// and, when the running max moved by more than 2^8, rescale O_t in tensor memory ->
// O_t += P_t V_j with P_t read from tensor memory as the A operand.
// The two row tiles alternate on the tensor core, so one tile's softmax overlaps
// the other's MMAs.
//
// Every wait is bounded (about two seconds): when one runs out the kernel sets a
// status word, all roles leave their loops, tensor memory is released and the
// kernel returns; the host turns the status into ELLM_ERR_DEVICE_TIMEOUT.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/ellm_attn.h"
#include "common.cuh"

namespace ellm {

constexpr int kTcTileRows = 128;   // rows per tile = tensor-memory lanes
constexpr int kTcTiles = 2;        // row tiles per CTA
constexpr int kTcKeys = 128;       // keys per K/V tile
constexpr int kTcStages = 5;       // ring slots, each holds one K or one V tile
constexpr int kTcTileBytes = kTcKeys * kRowBytes;          // 32 KB: two 16 KB halves of 128 rows x 128 B
constexpr int kTcHalfBytes = kTcTileBytes / 2;
constexpr int kTcThreads = (kTcTiles * 4 + 2) * 32;        // 320
constexpr int kTcSmemQ = 0;
constexpr int kTcSmemRing = kTcSmemQ + kTcTiles * kTcTileBytes;
constexpr int kTcSmemBar = kTcSmemRing + kTcStages * kTcTileBytes;
constexpr int kTcSmemBytes = kTcSmemBar + 256 + 1024;       // barriers + slack to align the base to 1024
constexpr float kTcRescaleThreshold = 8.0f;                 // log2 units
constexpr float kTcSumTrigger = 65536.0f;                   // a fast-path step whose row sum reaches this is redone with a rescale
#ifndef ELLM_TC_POLY_EVERY
#define ELLM_TC_POLY_EVERY 0
#endif
constexpr int kTcPolyEvery = ELLM_TC_POLY_EVERY;            // every n-th pair of a row uses the polynomial exp2 (0 = none)
constexpr int kTcPolyDiv = kTcPolyEvery > 0 ? kTcPolyEvery : 1;   // the divisor the selection below may use

struct Tcgen05Plan {
    bool ready = false;
    char why[160] = "";
    void* encode = nullptr;  // cuTensorMapEncodeTiled, fetched from the driver at run time
    int sm_count = 0;
    // the tensor maps of the last launch, reused when the next one has the same geometry
    CUtensorMap map_q, map_k, map_v, map_kn, map_vn;
    bool cached_fused = false;
    size_t cached_interval = 0, cached_batch = 0;
    long long cached_kv_rows = -1;
    const void* cached_q = nullptr;
    unsigned long long wait_timeout_ns = 2000000000ull;   // ellm_attn_set_option("tc_wait_timeout_ns")
    int debug_skip_item = -1;                              // ellm_attn_set_option("tc_debug_skip_kv_item")
    int persistent = -1;                                   // ellm_attn_set_option("tc_persistent"): -1 auto, 0 one CTA per item, 1 one CTA per SM
    int fuse_append = 1;                                   // ellm_attn_set_option("tc_fuse_append"): 0 keeps the separate append kernel
    int* sched = nullptr;                                  // the item counter and the exit counter of the one-CTA-per-SM form (the handle's)
};

struct TcParams {
    void* out;              // bf16, or fp32 for a partial result over a key window

    float* lse;
    int* status;            // device word: non-zero = a bounded wait ran out
    const int32_t* positions;  // per-sequence position of chunk row 0, or nullptr (then `base` for all)
    long long base;         // position of chunk row 0
    long long key_begin;    // rows attend keys [key_begin, min(position + 1, key_end)); key_end for a uniform chunk start only
    long long key_end;
    long long n_items;      // 256-row work items of the launch = pair_tiles * kv_heads * batch
    int* sched;             // two device words, zero between launches: [0] items handed out beyond the first
                            // one per CTA, [1] CTAs that have finished; nullptr = one item per CTA (grid = n_items)
    long long max_seq;      // rows per (sequence, kv head) in the cache
    int interval, batch, max_batch;
    int q_heads, kv_heads, group;
    int pair_tiles;         // 256-row CTA tiles per (sequence, kv head) = ceil(interval * group / 256)
    int pair_major;         // CTA order: 1 = all heads of the heaviest tile first, 0 = head by head
    unsigned long long wait_timeout_ns;   // bound of every device-side wait
    int debug_skip_item;    // test hook: ring item (K_0, V_0, K_1, ...) the producer never loads; -1 = none
    float scale_log2;
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done;
}

// Bounded wait.  Returns false when the CTA has been told to give up (abort word set by
// any thread) or when this wait itself ran out, in which case it sets both words.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_word, int* status,
                                            int code, unsigned long long timeout_ns) {
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_word) return false;
        if (global_timer_ns() - t0 > timeout_ns) {
            *abort_word = code;
            atomicCAS(status, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_word, int* status,
                                          int code, unsigned long long timeout_ns) {
    for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_word, status, code, timeout_ns);
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                            int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}

// shared -> global tile store of the same box shape (rows past the map's bound are dropped)
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle: rows of 128 bytes, 8-row groups
// `sbo` bytes apart, 64-element column blocks `lbo` bytes apart (used by MN-major operands).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>((lbo >> 4) & 0x3fffu) << 16;
    d |= static_cast<uint64_t>((sbo >> 4) & 0x3fffu) << 32;
    d |= 1ull << 46;   // descriptor version of this architecture
    d |= 2ull << 61;   // SWIZZLE_128B
    return d;
}
// Instruction descriptor: bf16 x bf16 -> fp32, M = 128, N = 128; b_mn_major selects a B
// operand whose N dimension is contiguous in shared memory.
__host__ __device__ constexpr uint32_t umma_idesc(bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((128u >> 3) << 17) |
           ((128u >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Same with the A operand in tensor memory (128 lanes x 8 columns of packed bf16 pairs per 16-wide K step).
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 consecutive fp32 columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32u(uint32_t taddr, const uint32_t* r);
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    tmem_st32u(taddr, reinterpret_cast<const uint32_t*>(v));
}
__device__ __forceinline__ void tmem_st32u(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- packed fp32 pair arithmetic and the exp2 helpers of the softmax passes ----
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
// 2^x for a pair, x <= ~8, without the exp2 unit: x = n + f with n = round(x) (magic-number
// add), 2^f from a degree-3 polynomial on [-0.5, 0.5] (max relative error 7.5e-5, below the
// bf16 rounding P gets anyway), 2^n added into the exponent field.
__device__ __forceinline__ uint64_t exp2_poly2(uint64_t x2) {
    float x0, x1;
    unpack2(x2, x0, x1);
    const uint64_t xc = pack2(fmaxf(x0, -126.0f), fmaxf(x1, -126.0f));
    const uint64_t magic = pack2(12582912.0f, 12582912.0f), neg_magic = pack2(-12582912.0f, -12582912.0f);
    const uint64_t r2 = add2(xc, magic);              // low mantissa bits now hold round(x)
    const uint64_t n2 = add2(r2, neg_magic);          // round(x) as a float
    const uint64_t f2 = fma2(n2, pack2(-1.0f, -1.0f), xc);
    uint64_t p2 = fma2(f2, pack2(0.0551716685295105f, 0.0551716685295105f), pack2(0.2426111251115799f, 0.2426111251115799f));
    p2 = fma2(p2, f2, pack2(0.6932609677314758f, 0.6932609677314758f));
    p2 = fma2(p2, f2, pack2(0.9999280571937561f, 0.9999280571937561f));
    float r0, r1, p0, p1;
    unpack2(r2, r0, r1);
    unpack2(p2, p0, p1);
    const float y0 = __int_as_float(__float_as_int(p0) + (__float_as_int(r0) << 23));
    const float y1 = __int_as_float(__float_as_int(p1) + (__float_as_int(r1) << 23));
    return pack2(y0, y1);
}

// Optional per-CTA time stamps for tuning (compiled in only with -DELLM_TC_TRACE): slot -> SM clock.
#ifdef ELLM_TC_TRACE
__device__ long long g_tc_trace[1024 * 64];
#define TC_TRACE(slot)                                                                   \
    do {                                                                                 \
        if (blockIdx.x < 1024 && (slot) < 64) g_tc_trace[blockIdx.x * 64 + (slot)] = clock64(); \
    } while (0)
#define TC_TRACE_NS(slot)                                                                \
    do {                                                                                 \
        if (blockIdx.x < 1024 && (slot) < 64) g_tc_trace[blockIdx.x * 64 + (slot)] = static_cast<long long>(global_timer_ns()); \
    } while (0)
#else
#define TC_TRACE(slot) do {} while (0)
#define TC_TRACE_NS(slot) do {} while (0)
#endif

// Status codes written by a wait that ran out (which wait gave up).
enum { kTcWaitQ = 1, kTcWaitKvFull = 2, kTcWaitKvEmpty = 3, kTcWaitSFull = 4, kTcWaitPFull = 5, kTcWaitPvDone = 6,
       kTcWaitQEmpty = 7, kTcWaitSched = 8 };

// One work item: 256 packed rows (two 128-row tiles) of one (sequence, KV head).
struct TcItem {
    int pair, kvh, b;
    long long base;      // position of the sequence's chunk row 0
    long long key_end;   // rows attend keys [key_begin, min(position + 1, key_end))
    int j0;              // first 128-key tile of the window
    int lo;              // first visible column of that tile (key_begin - 128 * j0)
    int steps[kTcTiles]; // key tiles row tile t needs (0: no valid row, or no key of the window in reach)
    int nsteps;
    bool zero_tail;
};

// The items are numbered heaviest first: later row tiles have more keys.  When all heads' K/V fit
// in L2 together the order is heaviest-first over the whole launch, else head by head so that one
// head's K/V stays resident while its row tiles are worked off.  A CTA starts with item blockIdx.x
// and then takes the next item nobody has taken yet (a device counter): long items first, short
// ones fill the ends, whatever the items turn out to cost.
__device__ __forceinline__ void tc_item(const TcParams& p, long long idx, TcItem& it) {
    const int heads = p.kv_heads * p.batch;
    int head;
    if (p.pair_major) {
        it.pair = p.pair_tiles - 1 - static_cast<int>(idx / heads);
        head = static_cast<int>(idx % heads);
    } else {
        head = static_cast<int>(idx / p.pair_tiles);
        it.pair = p.pair_tiles - 1 - static_cast<int>(idx % p.pair_tiles);
    }
    it.kvh = head % p.kv_heads;
    it.b = head / p.kv_heads;
    // where this sequence's chunk starts and where its keys end
    it.base = p.positions ? static_cast<long long>(p.positions[it.b]) : p.base;
    it.key_end = p.positions ? min(it.base + p.interval, p.max_seq) : p.key_end;
    it.j0 = static_cast<int>(p.key_begin / kTcKeys);
    it.lo = static_cast<int>(p.key_begin - static_cast<long long>(it.j0) * kTcKeys);
    const int total_rows = p.interval * p.group;
    it.nsteps = 0;
#pragma unroll
    for (int t = 0; t < kTcTiles; ++t) {
        const int rho0 = (it.pair * kTcTiles + t) * kTcTileRows;
        int s = 0;
        if (rho0 < total_rows) {
            const int rho_last = min(rho0 + kTcTileRows, total_rows) - 1;
            long long kend = it.base + rho_last / p.group + 1;
            if (kend > it.key_end) kend = it.key_end;
            s = static_cast<int>((kend + kTcKeys - 1) / kTcKeys) - it.j0;
            if (s < 0) s = 0;
        }
        it.steps[t] = s;
        it.nsteps = max(it.nsteps, s);
    }
    // With per-sequence chunk starts the K/V tensor maps are bounded by the cache, not by this
    // sequence's end, so the last V tile may carry rows past key_end that hold anything; their P
    // is 0 but 0 * NaN is NaN, so the producer zeroes them before the MMA may read the tile.
    it.zero_tail = p.positions != nullptr && static_cast<long long>(it.j0 + it.nsteps) * kTcKeys > it.key_end;
}

// A wait of the teardown: bounded, sets no status.
__device__ __noinline__ bool mbar_wait_quiet(uint32_t bar, uint32_t parity, unsigned long long timeout_ns) {
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > timeout_ns) return false;
    }
}

// Rare tail of the one-pass step: a score among the row's second 64 keys leapt far above the maximum in
// use after the first 64 keys' P had gone to tensor memory.  Finds the second half's true maximum,
// rescales O_t and the stored first half of P_t to it, and recomputes the second half.  Out of line:
// its registers must not be charged to the plain step.
struct TcFixed {
    float m_used, l;
};
__device__ __noinline__ TcFixed tc_fix_second_half(uint32_t tS, uint32_t tO, float scale_log2, float m_used, float l,
                                                   float first_half_sum, uint32_t* pk) {
    float mx = -INFINITY;
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
        float v[32];
        tmem_ld32(tS + 64 + c * 32, v);
        tmem_wait_ld();
        float m0 = max3(v[0], v[1], v[2]), m1 = max3(v[3], v[4], v[5]);
#pragma unroll
        for (int i = 6; i < 30; i += 6) {
            m0 = max3(m0, v[i], v[i + 1]);
            m1 = max3(m1, v[i + 2], v[i + 3]);
            m0 = fmaxf(m0, v[i + 4]);
            m1 = fmaxf(m1, v[i + 5]);
        }
        mx = max3(mx, max3(m0, v[30], v[31]), m1);
    }
    const float m_new = fmaxf(m_used, mx * scale_log2);
    // rows whose maximum did not move far keep it (their corr is 1): as in the two-pass step
    const bool moved = m_new - m_used > kTcRescaleThreshold;
    const float corr = moved ? fast_exp2(m_used - m_new) : 1.0f;
    if (moved) m_used = m_new;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {   // O_t: every P.V of earlier steps has completed (this step's S_t exists)
        float o[32];
        tmem_ld32(tO + c * 32, o);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] *= corr;
        tmem_st32(tO + c * 32, o);
    }
    {   // the first half of P_t, bf16 pairs in columns [0, 32)
        uint32_t q[32];
        tmem_ld32(tS, *reinterpret_cast<float(*)[32]>(&q[0]));
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&q[i]);
            q[i] = pack_bf16(__low2float(h) * corr, __high2float(h) * corr);
        }
        tmem_st32u(tS, q);
    }
    const uint64_t scale2 = pack2(scale_log2, scale_log2), negm2 = pack2(-m_used, -m_used);
    uint64_t sum_a = pack2(0.0f, 0.0f), sum_b = sum_a;
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
        float v[32];
        tmem_ld32(tS + 64 + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int cc = 0; cc < 16; ++cc) {
            const uint64_t x2 = fma2(pack2(v[2 * cc], v[2 * cc + 1]), scale2, negm2);
            float x0, x1;
            unpack2(x2, x0, x1);
            const uint64_t p2 = pack2(fast_exp2(x0), fast_exp2(x1));
            if (cc & 1) sum_b = add2(sum_b, p2); else sum_a = add2(sum_a, p2);
            float p0, p1;
            unpack2(p2, p0, p1);
            pk[c * 16 + cc] = pack_bf16(p0, p1);
        }
    }
    float sa, sb;
    unpack2(add2(sum_a, sum_b), sa, sb);
    TcFixed r;
    r.m_used = m_used;
    r.l = (l + first_half_sum) * corr + (sa + sb);
    return r;
}

// kFused: the chunk's own K/V rows come from k_new / v_new and are written into the cache here (a
// separate instantiation, so that the plain kernel carries none of its state).
template <typename OutT, bool kFused>
__global__ void __launch_bounds__(kTcThreads, 1)
prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_kn,
                       const __grid_constant__ CUtensorMap map_vn, const TcParams p) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) { TC_TRACE_NS(0); TC_TRACE(1); }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == (kTcTiles * 4) * 32) {   // the producer thread fetches the three descriptors ahead of its first copy
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
        if (kFused) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_kn) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_vn) : "memory");
        }
    }

    // barriers (8 bytes each) and two words behind them
    const uint32_t bar0 = smem_base + kTcSmemBar;
    auto bar_q = [&](int t) { return bar0 + 8u * t; };
    auto bar_kv_full = [&](int s) { return bar0 + 8u * (2 + s); };
    auto bar_kv_empty = [&](int s) { return bar0 + 8u * (2 + kTcStages + s); };
    auto bar_s_full = [&](int t) { return bar0 + 8u * (2 + 2 * kTcStages + t); };
    auto bar_p_full = [&](int t) { return bar0 + 8u * (4 + 2 * kTcStages + t); };
    auto bar_pv_done = [&](int t) { return bar0 + 8u * (6 + 2 * kTcStages + t); };
    auto bar_q_empty = [&](int t) { return bar0 + 8u * (8 + 2 * kTcStages + t); };
    const uint32_t bar_tail = bar0 + 8u * (10 + 2 * kTcStages);
    const uint32_t bar_final = bar0 + 8u * (11 + 2 * kTcStages);
    auto bar_sched_full = [&](int s) { return bar0 + 8u * (12 + 2 * kTcStages + s); };    // the item list's two-slot mailbox
    auto bar_sched_empty = [&](int s) { return bar0 + 8u * (14 + 2 * kTcStages + s); };
    constexpr int kNumBars = 16 + 2 * kTcStages;
    static_assert(8 * kNumBars + 24 <= 256, "the barrier block is 256 bytes");
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kTcSmemBar + 8 * kNumBars);
    volatile int* abort_word = reinterpret_cast<volatile int*>(smem + kTcSmemBar + 8 * kNumBars + 8);
    volatile int* sched_idx = reinterpret_cast<volatile int*>(smem + kTcSmemBar + 8 * kNumBars + 16);   // [2]

    if (threadIdx.x == 0) {
        for (int t = 0; t < kTcTiles; ++t) {
            mbar_init(bar_q(t), 1);
            mbar_init(bar_q_empty(t), 1);
            mbar_init(bar_s_full(t), 1);
            mbar_init(bar_p_full(t), kTcTileRows / 32);   // one arrival per softmax warp
            mbar_init(bar_pv_done(t), 1);
        }
        for (int s = 0; s < kTcStages; ++s) {
            mbar_init(bar_kv_full(s), 1);
            mbar_init(bar_kv_empty(s), 1);
        }
        mbar_init(bar_tail, 1);
        mbar_init(bar_final, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_sched_full(i), 1);
            mbar_init(bar_sched_empty(i), 1 + kTcTiles * 4);   // the MMA thread and every softmax warp
        }
        *abort_word = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kTcTiles * 4 + 1) {  // the MMA warp owns tensor memory: all 512 columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // columns: S_0 [0,128), S_1 [128,256), O_0 [256,384), O_1 [384,512)

    // Launched as a programmatic dependent, the set-up above ran while the stream's previous kernel
    // was still at work; everything below reads or writes what that kernel may have touched.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) TC_TRACE(2);
    const int total_rows = p.interval * p.group;
    const int n_items = static_cast<int>(p.n_items);
    // the k-th item of this CTA as the producer publishes it (n_items = no more)
    auto take_item = [&](long long k, bool& ok, int code) -> int {
        ok = mbar_wait(bar_sched_full(static_cast<int>(k & 1)), static_cast<uint32_t>((k >> 1) & 1), abort_word, p.status, code, p.wait_timeout_ns);
        const int idx = ok ? sched_idx[k & 1] : n_items;
        return idx;
    };

    // Every role walks the same list of items.  What carries over from one item to the next are the
    // barriers' phases, so each role counts what it has pushed through them so far: ring items,
    // key steps per row tile, Q loads per row tile, tail clean-ups.
    if (warp < kTcTiles * 4) {
        // =============================== softmax / correction / epilogue ===============================
        const int t = warp >> 2;
        const int row = (warp & 3) * 32 + lane;                 // row of the tile = tensor-memory lane
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tS = tmem + lane_base + t * 128;
        const uint32_t tO = tmem + lane_base + 256 + t * 128;
        int steps_done = 0;     // key steps of this row tile over all items so far
        bool ok = true;
        TcItem it;
        int n_traced = 0;
        for (long long k = 0; ok; ++k) {
            int idx = n_items;
            if (lane == 0) idx = take_item(k, ok, kTcWaitSched);
            idx = __shfl_sync(0xffffffffu, idx, 0);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            if (lane == 0) mbar_arrive(bar_sched_empty(static_cast<int>(k & 1)));
            if (idx >= n_items) break;
            tc_item(p, idx, it);
            const int tr = 8 + 8 * n_traced + 4 * t;   // trace slots of this item and tile
            ++n_traced;
            const int rho = (it.pair * kTcTiles + t) * kTcTileRows + row;
            const bool valid = rho < total_rows;
            const int pos = valid ? rho / p.group : 0, g = valid ? rho % p.group : 0;
            const long long lim = valid ? min(it.base + pos, it.key_end - 1) : -1;   // last key this row may see
            const long long tile_min_lim = min(it.base + ((it.pair * kTcTiles + t) * kTcTileRows) / p.group, it.key_end - 1);
            const int my_steps = it.steps[t];
            const long long row_index = (static_cast<long long>(pos) * p.max_batch + it.b) * p.q_heads + it.kvh * p.group + g;
            float m_used = -INFINITY, l = 0.0f;
            for (int j = 0; j < my_steps && ok; ++j) {
                // lane 0 polls the barrier, the warp follows (32 pollers per warp only add shared-memory traffic)
                ok = lane == 0 ? mbar_wait(bar_s_full(t), (steps_done + j) & 1, abort_word, p.status, kTcWaitSFull, p.wait_timeout_ns) : true;
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (j == 0 && (warp & 3) == 0 && lane == 0) TC_TRACE(tr);
                tc_fence_after();
                const long long key0 = static_cast<long long>(it.j0 + j) * kTcKeys;
                const int lo = j == 0 ? it.lo : 0;                     // columns below it lie before the key window
                const bool edge = key0 + kTcKeys - 1 > tile_min_lim || lo > 0;   // the causal edge (or the window's start) crosses this tile
                const long long dlim = lim - key0;                     // last column this row may see
                const int rel = dlim < 0 ? -1 : (dlim > 127 ? 127 : static_cast<int>(dlim));
                // Fast path (every step but the first, unless a score leaps far above the maximum in use):
                // exponentiate against the maximum already in use, in one pass.  P is held in registers
                // until the step's row sum has shown that nothing leapt - then it is consistent with O
                // and l as they stand and goes to tensor memory as is.  Otherwise S_t is still intact and
                // the two-pass slow path below redoes the step with a rescale of O_t.
                bool slow = (j == 0) || edge;
                if (!slow) {
                    // Half a row at a time: the first 64 keys' P goes to tensor memory (over columns of S_t
                    // that have been read) before the second 64 scores are fetched, so that a thread holds 64
                    // scores and 32 packed P values at most.
                    const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), negm2 = pack2(-m_used, -m_used);
                    uint32_t pk[32];
                    float half_sum[2];
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        float s[64];
                        tmem_ld32(tS + half * 64, *reinterpret_cast<float(*)[32]>(&s[0]));
                        tmem_ld32(tS + half * 64 + 32, *reinterpret_cast<float(*)[32]>(&s[32]));
                        tmem_wait_ld();
                        uint64_t sum_a = pack2(0.0f, 0.0f), sum_b = sum_a;
#pragma unroll
                        for (int cc = 0; cc < 32; ++cc) {
                            const uint64_t x2 = fma2(pack2(s[2 * cc], s[2 * cc + 1]), scale2, negm2);
                            uint64_t p2;
                            if (kTcPolyEvery > 0 && (cc % kTcPolyDiv) == kTcPolyDiv - 1) {
                                p2 = exp2_poly2(x2);
                            } else {
                                float x0, x1;
                                unpack2(x2, x0, x1);
                                p2 = pack2(fast_exp2(x0), fast_exp2(x1));
                            }
                            if (cc & 1) sum_b = add2(sum_b, p2); else sum_a = add2(sum_a, p2);
                            float p0, p1;
                            unpack2(p2, p0, p1);
                            pk[cc] = pack_bf16(p0, p1);
                        }
                        float sa, sb;
                        unpack2(add2(sum_a, sum_b), sa, sb);
                        half_sum[half] = sa + sb;
                        // No row maximum is tracked here.  A score far above the maximum in use shows up as a huge
                        // term of the sum (2^16 and more: one key 16 octaves above, or infinity).
                        const bool leapt = __any_sync(0xffffffffu, !(half_sum[half] < kTcSumTrigger));
                        if (half == 0) {
                            if (leapt) {   // S_t is still intact: the whole step the slow way
                                slow = true;
                                break;
                            }
                            tmem_st32u(tS, pk);
                        } else {
                            if (leapt) {   // the first half's P is already in place: bring it and O_t to the new maximum
                                uint32_t redone[32];   // (addressable only here: pk itself stays in registers)
                                const TcFixed f = tc_fix_second_half(tS, tO, p.scale_log2, m_used, l, half_sum[0], redone);
                                m_used = f.m_used;
                                l = f.l;
#pragma unroll
                                for (int i = 0; i < 32; ++i) pk[i] = redone[i];
                            } else {
                                l += half_sum[0] + half_sum[1];
                            }
                            tmem_st32u(tS + 32, pk);
                            tmem_wait_st();
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(bar_p_full(t));
                        }
                    }
                }
                if (slow) {
                    // pass 1 over S_t: row maximum (3-input max, two chains per 32-column chunk).  The
                    // scores are read again in pass 2 rather than kept: tensor-memory reads are cheap and
                    // 128 live registers per thread are not.
                    float mx = -INFINITY;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float s[64];
                        tmem_ld32(tS + h * 64, *reinterpret_cast<float(*)[32]>(&s[0]));
                        tmem_ld32(tS + h * 64 + 32, *reinterpret_cast<float(*)[32]>(&s[32]));
                        tmem_wait_ld();
                        if (edge) {
#pragma unroll
                            for (int c = 0; c < 64; ++c) s[c] = (h * 64 + c <= rel && h * 64 + c >= lo) ? s[c] : -INFINITY;
                        }
                        float m0 = max3(s[0], s[1], s[2]), m1 = max3(s[3], s[4], s[5]);
                        float m2 = max3(s[6], s[7], s[8]), m3 = max3(s[9], s[10], s[11]);
#pragma unroll
                        for (int c = 12; c < 60; c += 8) {
                            m0 = max3(m0, s[c], s[c + 1]);
                            m1 = max3(m1, s[c + 2], s[c + 3]);
                            m2 = max3(m2, s[c + 4], s[c + 5]);
                            m3 = max3(m3, s[c + 6], s[c + 7]);
                        }
                        m0 = max3(m0, s[60], s[61]);
                        m1 = max3(m1, s[62], s[63]);
                        mx = max3(mx, fmaxf(m0, m1), fmaxf(m2, m3));
                    }
                    const float m_new = fmaxf(m_used, mx * p.scale_log2);
                    // rescale O only when the maximum moved far enough to matter; otherwise keep
                    // exponentiating against the stale maximum (O and l stay consistent with it)
                    const bool need = (m_new - m_used > kTcRescaleThreshold) || (m_used == -INFINITY && m_new != -INFINITY);
                    const bool rescale = __any_sync(0xffffffffu, need);
                    float corr = 1.0f;
                    if (rescale) {
                        corr = (m_used == -INFINITY) ? 0.0f : fast_exp2(m_used - m_new);
                        m_used = m_new;
                    }
                    const float msub = (m_used == -INFINITY) ? 0.0f : m_used;
                    // S_t(j) complete implies P.V(t, j-1) complete (MMAs of one thread finish in issue
                    // order), so O_t can be rescaled and the columns of S_t can take P_t right away.
                    if (rescale && j > 0) {   // before any P.V of this step may start
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            float o[32];
                            tmem_ld32(tO + c * 32, o);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] *= corr;
                            tmem_st32(tO + c * 32, o);
                        }
                    }
                    // pass 2: p = exp2(s * scale - m) on packed pairs; P row -> tensor memory as bf16
                    // pairs (k, k+1) per 32-bit column, 64 columns, over the first half of S_t.
                    {
                        const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), negm2 = pack2(-msub, -msub);
                        uint64_t sum_a = pack2(0.0f, 0.0f), sum_b = sum_a;
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            // keys [64*half, 64*half+64) of S sit in columns [64*half, +64); their P goes to
                            // columns [32*half, +32), which never overlap a half of S not yet read
                            float s[64];
                            tmem_ld32(tS + half * 64, *reinterpret_cast<float(*)[32]>(&s[0]));
                            tmem_ld32(tS + half * 64 + 32, *reinterpret_cast<float(*)[32]>(&s[32]));
                            tmem_wait_ld();
                            if (edge) {
#pragma unroll
                                for (int c = 0; c < 64; ++c) s[c] = (half * 64 + c <= rel && half * 64 + c >= lo) ? s[c] : -INFINITY;
                            }
                            uint32_t pk[32];
#pragma unroll
                            for (int cc = 0; cc < 32; ++cc) {
                                const int c = half * 32 + cc;
                                const uint64_t x2 = fma2(pack2(s[2 * cc], s[2 * cc + 1]), scale2, negm2);
                                uint64_t p2;
                                if (kTcPolyEvery > 0 && (c % kTcPolyDiv) == kTcPolyDiv - 1) {
                                    p2 = exp2_poly2(x2);
                                } else {
                                    float x0, x1;
                                    unpack2(x2, x0, x1);
                                    p2 = pack2(fast_exp2(x0), fast_exp2(x1));
                                }
                                if (c & 1) sum_b = add2(sum_b, p2); else sum_a = add2(sum_a, p2);
                                float p0, p1;
                                unpack2(p2, p0, p1);
                                pk[cc] = pack_bf16(p0, p1);
                            }
                            tmem_st32u(tS + half * 32, pk);
                            tmem_wait_st();
                            tc_fence_before();
                            __syncwarp();
                            if (half == 1 && lane == 0) mbar_arrive(bar_p_full(t));
                        }
                        float sa, sb;
                        unpack2(add2(sum_a, sum_b), sa, sb);
                        l = l * corr + (sa + sb);
                    }
                }
            }
            if ((warp & 3) == 0 && lane == 0) TC_TRACE(tr + 1);
            if (ok && my_steps > 0) {
                ok = mbar_wait(bar_pv_done(t), (steps_done + my_steps - 1) & 1, abort_word, p.status, kTcWaitPvDone, p.wait_timeout_ns);
                ok = __all_sync(0xffffffffu, ok);
            }
            if (!ok) break;
            if ((warp & 3) == 0 && lane == 0) TC_TRACE(tr + 2);
            OutT* orow = reinterpret_cast<OutT*>(p.out) + row_index * kHeadDim;
            if (my_steps > 0) {
                tc_fence_after();
                const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float o[32];
                    tmem_ld32(tO + c * 32, o);
                    tmem_wait_ld();
                    if (valid) {
                        if constexpr (sizeof(OutT) == 4) {
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                *reinterpret_cast<float4*>(orow + c * 32 + i * 4) =
                                    make_float4(o[i * 4 + 0] * inv, o[i * 4 + 1] * inv, o[i * 4 + 2] * inv, o[i * 4 + 3] * inv);
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                uint4 v;
                                v.x = pack_bf16(o[i * 8 + 0] * inv, o[i * 8 + 1] * inv);
                                v.y = pack_bf16(o[i * 8 + 2] * inv, o[i * 8 + 3] * inv);
                                v.z = pack_bf16(o[i * 8 + 4] * inv, o[i * 8 + 5] * inv);
                                v.w = pack_bf16(o[i * 8 + 6] * inv, o[i * 8 + 7] * inv);
                                *reinterpret_cast<uint4*>(orow + c * 32 + i * 8) = v;
                            }
                        }
                    }
                }
                if (valid && p.lse) p.lse[row_index] = (m_used + log2f(l)) * kLn2;
                // the next item's first P.V overwrites O_t: its P is only handed over by these same
                // threads, after the reads above have completed
                tc_fence_before();
            } else if (valid) {
                // no key of the window lies in reach of this tile's rows: an empty partial result
                if constexpr (sizeof(OutT) == 4) {
                    for (int i = 0; i < 32; ++i) *reinterpret_cast<float4*>(orow + i * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
                } else {
                    for (int i = 0; i < 16; ++i) *reinterpret_cast<uint4*>(orow + i * 8) = make_uint4(0u, 0u, 0u, 0u);
                }
                if (p.lse) p.lse[row_index] = -INFINITY;
            }
            steps_done += my_steps;
            if ((warp & 3) == 0 && lane == 0) TC_TRACE(tr + 3);
        }
    } else if (warp == kTcTiles * 4) {
        // =============================== TMA producer ===============================
        if (lane == 0) {
            bool ok = true;
            long long ring_n = 0;                   // ring items requested so far (K_0, V_0, K_1, ... of every item)
            int q_loads[kTcTiles] = {0, 0};
            int tails = 0;
            // fused append: tiles waiting to be stored into the cache, per ring slot
            bool store_pending[kTcStages] = {};
            long long store_ring[kTcStages] = {};
            int store_key0[kTcStages] = {};
            int store_head[kTcStages] = {};
            // waits until the slot's tile has landed, stores it to the cache rows it holds and waits until the
            // store has read the slot (so that the slot can be refilled)
            auto flush_store = [&](int slot) -> bool {
                const long long r = store_ring[slot];
                if (!mbar_wait(bar_kv_full(slot), static_cast<uint32_t>((r / kTcStages) & 1), abort_word, p.status, kTcWaitKvFull, p.wait_timeout_ns))
                    return false;
                const int hd = store_head[slot];
                const CUtensorMap* map = (hd >> 30) ? &map_v : &map_k;
                for (int h = 0; h < 2; ++h)
                    tma_store_4d(map, smem_base + kTcSmemRing + slot * kTcTileBytes + h * kTcHalfBytes, h * 64, store_key0[slot],
                                 hd & 0xffff, (hd >> 16) & 0x3fff);
                bulk_commit();
                bulk_wait_read_all();
                store_pending[slot] = false;
                return true;
            };
            TcItem it;
            for (long long k = 0; ok; ++k) {
                // this CTA's k-th item: its own block index first, then whatever comes next on the list
                long long idx = blockIdx.x;
                if (k > 0) idx = p.sched ? static_cast<long long>(gridDim.x) + atomicAdd(p.sched, 1) : p.n_items;
                if (idx > p.n_items) idx = p.n_items;
                ok = mbar_wait(bar_sched_empty(static_cast<int>(k & 1)), static_cast<uint32_t>(((k >> 1) & 1) ^ 1), abort_word, p.status,
                               kTcWaitSched, p.wait_timeout_ns);
                if (!ok) break;
                sched_idx[k & 1] = static_cast<int>(idx);
                mbar_arrive(bar_sched_full(static_cast<int>(k & 1)));   // releases the word above to the waiters
                if (idx >= p.n_items) break;
                tc_item(p, idx, it);
                for (int t = 0; t < kTcTiles && ok; ++t) {
                    if (it.steps[t] == 0) continue;
                    // the previous item's last Q.K^T of this row tile has finished with the Q tile
                    ok = mbar_wait(bar_q_empty(t), (q_loads[t] & 1) ^ 1, abort_word, p.status, kTcWaitQEmpty, p.wait_timeout_ns);
                    if (!ok) break;
                    const int rho0 = (it.pair * kTcTiles + t) * kTcTileRows;
                    mbar_arrive_expect_tx(bar_q(t), kTcTileBytes);
                    for (int h = 0; h < 2; ++h)
                        tma_load_5d(smem_base + kTcSmemQ + t * kTcTileBytes + h * kTcHalfBytes, &map_q, bar_q(t), h * 64, 0,
                                    rho0 / p.group, it.kvh, it.b);
                    ++q_loads[t];
                }
                for (int item = 0; item < 2 * it.nsteps && ok; ++item, ++ring_n) {  // K_0, V_0, K_1, V_1, ...
                    const int slot = static_cast<int>(ring_n % kTcStages);
                    const uint32_t round_par = static_cast<uint32_t>((ring_n / kTcStages) & 1);
                    if constexpr (kFused) {
                        // a tile of the chunk's own rows that waits in this slot to be written into the cache
                        // goes out first (it landed long ago: the slot has been consumed since)
                        if (store_pending[slot]) ok = flush_store(slot);
                        if (!ok) break;
                    }
                    ok = mbar_wait(bar_kv_empty(slot), round_par ^ 1, abort_word, p.status, kTcWaitKvEmpty, p.wait_timeout_ns);
                    if (!ok) break;
                    if (ring_n == p.debug_skip_item) continue;   // test hook: this item's barrier is never signalled
                    const int key0 = (it.j0 + (item >> 1)) * kTcKeys;
                    if constexpr (kFused) {
                        // Key tiles at or past the chunk's start hold the chunk's own rows, which are not in the
                        // cache yet - they come from k_new / v_new (row = key - chunk start).  Exactly one item
                        // writes such a tile into the cache: the one whose rows include the tile's first token.
                        const bool from_new = key0 >= p.base;
                        const CUtensorMap* map = from_new ? ((item & 1) ? &map_vn : &map_kn) : ((item & 1) ? &map_v : &map_k);
                        const int row0 = from_new ? key0 - static_cast<int>(p.base) : key0;
                        mbar_arrive_expect_tx(bar_kv_full(slot), kTcTileBytes);
                        for (int h = 0; h < 2; ++h)
                            tma_load_4d(smem_base + kTcSmemRing + slot * kTcTileBytes + h * kTcHalfBytes, map, bar_kv_full(slot),
                                        h * 64, row0, it.kvh, it.b);
                        if (from_new && (static_cast<long long>(row0 / kTcKeys) * p.group) / 2 == it.pair) {
                            store_pending[slot] = true;
                            store_ring[slot] = ring_n;
                            store_key0[slot] = key0;
                            store_head[slot] = it.kvh | (it.b << 16) | ((item & 1) << 30);
                        }
                    } else {
                        const CUtensorMap* map = (item & 1) ? &map_v : &map_k;
                        mbar_arrive_expect_tx(bar_kv_full(slot), kTcTileBytes);
                        for (int h = 0; h < 2; ++h)
                            tma_load_4d(smem_base + kTcSmemRing + slot * kTcTileBytes + h * kTcHalfBytes, map, bar_kv_full(slot),
                                        h * 64, key0, it.kvh, it.b);
                    }
                }
                if (ok && it.zero_tail && it.nsteps > 0) {
                    const long long last = ring_n - 1;   // the last V tile
                    const int slot = static_cast<int>(last % kTcStages);
                    ok = mbar_wait(bar_kv_full(slot), static_cast<uint32_t>((last / kTcStages) & 1), abort_word, p.status, kTcWaitKvFull,
                                   p.wait_timeout_ns);
                    if (ok) {
                        // a 128-byte row of either half holds one key; the swizzle only permutes inside a row
                        const int first = static_cast<int>(it.key_end - static_cast<long long>(it.j0 + it.nsteps - 1) * kTcKeys);
                        unsigned char* tile = smem + kTcSmemRing + slot * kTcTileBytes;
                        for (int r = first; r < kTcKeys; ++r)
                            for (int h = 0; h < 2; ++h) {
                                uint4* rowp = reinterpret_cast<uint4*>(tile + h * kTcHalfBytes + r * 128);
#pragma unroll
                                for (int c = 0; c < 8; ++c) rowp[c] = make_uint4(0u, 0u, 0u, 0u);
                            }
                        fence_async_smem();
                        mbar_arrive(bar_tail);
                        ++tails;
                    }
                }
            }
            if (kFused) {
                for (int s = 0; s < kTcStages && ok; ++s)
                    if (store_pending[s]) ok = flush_store(s);
                bulk_wait_all();   // the cache rows are written before the kernel ends
            }
            if (*abort_word) {
                // a wait ran out somewhere: copies this thread requested may still be on their way into
                // shared memory.  Wait (bounded, quietly) for the barrier of every slot it armed last.
                for (int s = 0; s < kTcStages; ++s) {
                    const long long last = ring_n - 1 - ((ring_n - 1 - s) % kTcStages + kTcStages) % kTcStages;   // last item of slot s
                    if (last >= 0 && last != p.debug_skip_item)
                        mbar_wait_quiet(bar_kv_full(s), static_cast<uint32_t>((last / kTcStages) & 1), 200000ull);
                }
                for (int t = 0; t < kTcTiles; ++t)
                    if (q_loads[t] > 0) mbar_wait_quiet(bar_q(t), static_cast<uint32_t>((q_loads[t] - 1) & 1), 200000ull);
            }
            (void)tails;
        }
        __syncwarp();
    } else {
        // =============================== MMA issuer ===============================
        // One thread issues every MMA, one GEMM after the other: two issuing threads were tried and
        // lost 20 % because their GEMMs interleave on the tensor pipe and both finish late.
        if (lane == 0) {
            bool ok = true;
            constexpr uint32_t idesc_qk = umma_idesc(false), idesc_pv = umma_idesc(true);
            auto issue_qk = [&](int t, int slot) {  // S_t = Q_t K^T: 8 steps of 16 over head_dim
                const uint32_t q_addr = smem_base + kTcSmemQ + t * kTcTileBytes;
                const uint32_t k_addr = smem_base + kTcSmemRing + slot * kTcTileBytes;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (ks >> 2) * kTcHalfBytes + (ks & 3) * 32;
                    umma_bf16(tmem + t * 128, umma_desc(q_addr + off, 0, 1024), umma_desc(k_addr + off, 0, 1024), idesc_qk,
                              ks > 0);
                }
                umma_commit(bar_s_full(t));
            };
            // O_t += P_t V for keys [64*half, 64*half + 64): 4 steps of 16 keys
            auto issue_pv_half = [&](int t, int slot, bool first, int half) {
                const uint32_t v_addr = smem_base + kTcSmemRing + slot * kTcTileBytes;
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) {
                    const int ks = half * 4 + k4;
                    const uint32_t b_off = ks * 16 * 128;  // 16 key rows of 128 bytes
                    umma_bf16_a_tmem(tmem + 256 + t * 128, tmem + t * 128 + ks * 8,
                                     umma_desc(v_addr + b_off, kTcHalfBytes, 1024), idesc_pv, !(first && ks == 0));
                }
                if (half == 1) umma_commit(bar_pv_done(t));
            };
            long long ring_c = 0;                  // ring items of all earlier work items
            int steps_done[kTcTiles] = {0, 0};
            int q_loads[kTcTiles] = {0, 0};
            int tails = 0;
            TcItem it;
            for (long long k = 0; ok; ++k) {
                const int idx = take_item(k, ok, kTcWaitSched);
                if (!ok) break;
                mbar_arrive(bar_sched_empty(static_cast<int>(k & 1)));
                if (idx >= n_items) break;
                tc_item(p, idx, it);
                const int nsteps = it.nsteps;
                // ring item i of this work item: K_(i/2) for even i, V_(i/2) for odd i
                auto wait_item = [&](int item) {
                    const long long r = ring_c + item;
                    if (it.zero_tail && item == 2 * nsteps - 1)   // the last V tile is released by the producer's clean-up
                        return mbar_wait(bar_tail, static_cast<uint32_t>(tails & 1), abort_word, p.status, kTcWaitKvFull, p.wait_timeout_ns);
                    return mbar_wait(bar_kv_full(static_cast<int>(r % kTcStages)), static_cast<uint32_t>((r / kTcStages) & 1), abort_word,
                                     p.status, kTcWaitKvFull, p.wait_timeout_ns);
                };
                auto slot_of = [&](int item) { return static_cast<int>((ring_c + item) % kTcStages); };
                for (int t = 0; t < kTcTiles && ok; ++t)
                    if (it.steps[t] > 0) ok = mbar_wait(bar_q(t), static_cast<uint32_t>(q_loads[t] & 1), abort_word, p.status, kTcWaitQ, p.wait_timeout_ns);
                if (ok && nsteps > 0) {
                    ok = wait_item(0);
                    if (ok) {
                        tc_fence_after();
                        for (int t = 0; t < kTcTiles; ++t)
                            if (it.steps[t] > 0) {
                                issue_qk(t, slot_of(0));
                                if (it.steps[t] == 1) umma_commit(bar_q_empty(t));   // this item reads Q_t no more
                            }
                        umma_commit(bar_kv_empty(slot_of(0)));
                    }
                }
                for (int j = 0; j < nsteps && ok; ++j) {
                    const int item_v = 2 * j + 1, slot_v = slot_of(item_v);
                    const int item_k = 2 * j + 2, slot_k = slot_of(item_k);
                    bool have_v = false, have_k = false;
                    for (int t = 0; t < kTcTiles && ok; ++t) {
                        if (j >= it.steps[t]) continue;
                        ok = mbar_wait(bar_p_full(t), static_cast<uint32_t>((steps_done[t] + j) & 1), abort_word, p.status, kTcWaitPFull,
                                       p.wait_timeout_ns);
                        if (!ok) break;
                        if (!have_v) {
                            ok = wait_item(item_v);
                            if (!ok) break;
                            have_v = true;
                        }
                        tc_fence_after();
                        issue_pv_half(t, slot_v, j == 0, 0);
                        issue_pv_half(t, slot_v, j == 0, 1);
                        if (j + 1 < it.steps[t]) {
                            if (!have_k) {
                                ok = wait_item(item_k);
                                if (!ok) break;
                                have_k = true;
                                tc_fence_after();
                            }
                            issue_qk(t, slot_k);
                            if (j + 2 == it.steps[t]) umma_commit(bar_q_empty(t));
                        }
                    }
                    if (!ok) break;
                    umma_commit(bar_kv_empty(slot_v));                      // V_j free once every MMA so far is done
                    if (j + 1 < nsteps) umma_commit(bar_kv_empty(slot_k));  // and K_{j+1}
                }
                if (!ok) break;
                ring_c += 2 * nsteps;
                if (it.zero_tail && nsteps > 0) ++tails;
                for (int t = 0; t < kTcTiles; ++t) {
                    steps_done[t] += it.steps[t];
                    if (it.steps[t] > 0) ++q_loads[t];
                }
            }
            // every MMA issued above has completed before tensor memory is given back
            umma_commit(bar_final);
            mbar_wait_quiet(bar_final, 0, *abort_word ? 2000000ull : p.wait_timeout_ns);
        }
        __syncwarp();
    }

    // teardown: every role gets here (all waits are bounded)
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) { TC_TRACE(3); TC_TRACE_NS(4); }
    if (threadIdx.x == 0 && p.sched) {
        // the last CTA to leave puts the two words back to zero for the next launch
        __threadfence();
        if (atomicAdd(p.sched + 1, 1) == static_cast<int>(gridDim.x) - 1) {
            p.sched[0] = 0;
            p.sched[1] = 0;
            __threadfence();
        }
    }
    if (warp == kTcTiles * 4 + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
    }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline void tcgen05_plan_init(Tcgen05Plan& plan, const ellm_attn_desc& d, int sm_count) {
    plan.ready = false;
    plan.sm_count = sm_count;
    const size_t group = d.q_heads / d.kv_heads;
    if (group > 128 || (128 % group) != 0) {
        snprintf(plan.why, sizeof(plan.why), "query heads per KV head (%zu) must divide 128", group);
        return;
    }
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn ||
        qres != cudaDriverEntryPointSuccess) {
        cudaGetLastError();
        snprintf(plan.why, sizeof(plan.why), "driver does not export cuTensorMapEncodeTiled");
        return;
    }
    if (cudaFuncSetAttribute(prefill_tcgen05_kernel<__nv_bfloat16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(prefill_tcgen05_kernel<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(prefill_tcgen05_kernel<float, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes) != cudaSuccess) {
        snprintf(plan.why, sizeof(plan.why), "cannot reserve %d bytes of shared memory: %s", kTcSmemBytes,
                 cudaGetErrorString(cudaGetLastError()));
        return;
    }
    plan.encode = fn;
    plan.ready = true;
}

// AUTO picks this kernel for every chunk of at least 16 packed rows (rows x query heads of a
// group); a shorter chunk leaves more than 7/8 of a 128-row tile empty and goes to the warp-level kernel.
inline bool tcgen05_prefers(const Tcgen05Plan& plan, size_t interval, int group) {
    return plan.ready && interval * static_cast<size_t>(group) >= 16;
}

// The append can ride in the kernel when the chunk starts on a 128-key tile boundary with one start
// for all sequences and the whole key range is attended: then every key tile holds either cache rows
// only or new rows only.
inline bool tcgen05_can_fuse_append(const Tcgen05Plan& plan, const ellm_attn_desc& d, const int32_t* positions,
                                    size_t position_index, size_t batch, long long key_begin, long long key_end) {
    return plan.ready && plan.fuse_append && d.k_new && d.v_new && !positions && position_index % kTcKeys == 0 && key_begin == 0 &&
           key_end >= static_cast<long long>(d.max_seq) && batch < 16384 && d.kv_heads < 65536 &&
           (d.max_batch * d.kv_heads * 256) % 16 == 0;
}

// With a uniform chunk start the K/V tensor maps are bounded at min(position_index + interval,
// key_end) so that TMA zero-fills rows the chunk must not read; with per-sequence starts
// (positions != nullptr) they are bounded by the cache and the kernel zeroes the tail itself.
// out_f32 != nullptr writes an fp32 partial result there instead of bf16 to d.out.
inline int launch_prefill_tcgen05(Tcgen05Plan& plan, const ellm_attn_desc& d, const int32_t* positions,
                                  size_t position_index, size_t interval, size_t batch, long long key_begin,
                                  long long key_end, float* out_f32, float* lse, int* status, cudaStream_t stream,
                                  bool fused_append = false) {
    if (!plan.ready) return ELLM_ERR_UNSUPPORTED;
    const int group = static_cast<int>(d.q_heads / d.kv_heads);
    // per-sequence chunk starts: the maps can only be bounded by the cache itself
    long long kv_rows = positions ? static_cast<long long>(d.max_seq) : static_cast<long long>(position_index + interval);
    if (kv_rows > key_end) kv_rows = key_end;
    if (kv_rows > static_cast<long long>(d.max_seq)) kv_rows = static_cast<long long>(d.max_seq);
    if (kv_rows <= 0 || key_begin < 0 || (positions && key_begin != 0)) {
        snprintf(plan.why, sizeof(plan.why), "empty key window, or a window start together with per-sequence positions");
        return ELLM_ERR_UNSUPPORTED;
    }
    EncodeTiledFn encode = reinterpret_cast<EncodeTiledFn>(plan.encode);
    CUtensorMap& map_q = plan.map_q;
    CUtensorMap& map_k = plan.map_k;
    CUtensorMap& map_v = plan.map_v;
    // the buffers, head counts and strides are fixed for the handle: the maps depend only on these
    const bool reuse = plan.cached_kv_rows == kv_rows && plan.cached_interval == interval && plan.cached_batch == batch &&
                       plan.cached_q == d.q && plan.cached_fused == fused_append;
    plan.cached_kv_rows = -1;
    if (!reuse) {
        // q viewed as [head_dim, g, chunk row, kv head, sequence]; a box is 64 x G x (128/G) packed rows
        cuuint64_t dims[5] = {128, static_cast<cuuint64_t>(group), interval, d.kv_heads, d.max_batch};
        cuuint64_t strides[4] = {256, d.max_batch * d.q_heads * 256, static_cast<cuuint64_t>(group) * 256, d.q_heads * 256};
        cuuint32_t box[5] = {64, static_cast<cuuint32_t>(group), static_cast<cuuint32_t>(128 / group), 1, 1};
        cuuint32_t es[5] = {1, 1, 1, 1, 1};
        if (encode(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(d.q), dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
            snprintf(plan.why, sizeof(plan.why), "cuTensorMapEncodeTiled(q) failed");
            return ELLM_ERR_UNSUPPORTED;
        }
    }
    for (int which = 0; which < 2 && !reuse; ++which) {
        cuuint64_t dims[4] = {128, static_cast<cuuint64_t>(kv_rows), d.kv_heads, batch};
        cuuint64_t strides[3] = {d.kv_strides[2] * 2, d.kv_strides[1] * 2, d.kv_strides[0] * 2};
        cuuint32_t box[4] = {64, 128, 1, 1};
        cuuint32_t es[4] = {1, 1, 1, 1};
        if (encode(which ? &map_v : &map_k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, which ? d.v_cache : d.k_cache, dims,
                   strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
            snprintf(plan.why, sizeof(plan.why), "cuTensorMapEncodeTiled(k/v) failed");
            return ELLM_ERR_UNSUPPORTED;
        }
    }
    if (fused_append && !reuse) {
        // the chunk's new rows [chunk row, sequence, kv head, 128] seen as (128, chunk row, kv head, sequence):
        // the same box as a cache tile, so a tile of new rows lands in shared memory exactly like a cache tile
        for (int which = 0; which < 2; ++which) {
            cuuint64_t dims[4] = {128, interval, d.kv_heads, batch};
            cuuint64_t strides[3] = {d.max_batch * d.kv_heads * 256, 256, d.kv_heads * 256};
            cuuint32_t box[4] = {64, 128, 1, 1};
            cuuint32_t es[4] = {1, 1, 1, 1};
            if (encode(which ? &plan.map_vn : &plan.map_kn, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                       const_cast<void*>(which ? d.v_new : d.k_new), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
                snprintf(plan.why, sizeof(plan.why), "cuTensorMapEncodeTiled(k_new / v_new) failed");
                return ELLM_ERR_UNSUPPORTED;
            }
        }
    }
    plan.cached_fused = fused_append;
    plan.cached_kv_rows = kv_rows;
    plan.cached_interval = interval;
    plan.cached_batch = batch;
    plan.cached_q = d.q;
    TcParams p;
    p.out = out_f32 ? static_cast<void*>(out_f32) : d.out;
    p.key_begin = key_begin;
    p.key_end = kv_rows;
    p.lse = lse;
    p.status = status;
    p.base = static_cast<long long>(position_index);
    p.positions = positions;
    p.max_seq = static_cast<long long>(d.max_seq);
    p.wait_timeout_ns = plan.wait_timeout_ns;
    p.debug_skip_item = plan.debug_skip_item;
    p.interval = static_cast<int>(interval);
    p.batch = static_cast<int>(batch);
    p.max_batch = static_cast<int>(d.max_batch);
    p.q_heads = static_cast<int>(d.q_heads);
    p.kv_heads = static_cast<int>(d.kv_heads);
    p.group = group;
    p.pair_tiles = static_cast<int>((interval * group + kTcTiles * kTcTileRows - 1) / (kTcTiles * kTcTileRows));
    p.scale_log2 = d.scale * kLog2e;
    const unsigned long long items = static_cast<unsigned long long>(p.pair_tiles) * p.kv_heads * p.batch;
    if (items > 0x7fffffffull) {
        snprintf(plan.why, sizeof(plan.why), "too many row tiles for one launch");
        return ELLM_ERR_UNSUPPORTED;
    }
    p.n_items = static_cast<long long>(items);
    // One CTA per SM walking the item list (no second wave that starts from nothing, the set-up paid
    // once), or one CTA per item taken by the hardware in block order.
    const bool persistent = plan.sched != nullptr && (plan.persistent < 0 ? true : plan.persistent != 0);
    const unsigned long long ctas = persistent ? std::min<unsigned long long>(items, static_cast<unsigned long long>(plan.sm_count)) : items;
    p.sched = persistent ? plan.sched : nullptr;
    // K and V rows this launch can touch, all heads and sequences together
    const unsigned long long kv_bytes = 2ull * static_cast<unsigned long long>(kv_rows) * 256ull * d.kv_heads * batch;
    p.pair_major = kv_bytes <= (96ull << 20) ? 1 : 0;
    // a programmatic dependent of the stream's previous kernel: set-up overlaps that kernel's tail
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(ctas));
    cfg.blockDim = dim3(kTcThreads);
    cfg.dynamicSmemBytes = kTcSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // without the fused append the two extra maps are never used; any valid map will do
    const CUtensorMap& map_kn = fused_append ? plan.map_kn : map_k;
    const CUtensorMap& map_vn = fused_append ? plan.map_vn : map_v;
    if (fused_append && out_f32) {
        snprintf(plan.why, sizeof(plan.why), "the fused append comes with bf16 output only");
        return ELLM_ERR_UNSUPPORTED;
    }
    const cudaError_t e =
        out_f32        ? cudaLaunchKernelEx(&cfg, prefill_tcgen05_kernel<float, false>, map_q, map_k, map_v, map_kn, map_vn, p)
        : fused_append ? cudaLaunchKernelEx(&cfg, prefill_tcgen05_kernel<__nv_bfloat16, true>, map_q, map_k, map_v, map_kn, map_vn, p)
                       : cudaLaunchKernelEx(&cfg, prefill_tcgen05_kernel<__nv_bfloat16, false>, map_q, map_k, map_v, map_kn, map_vn, p);
    return e == cudaSuccess ? ELLM_OK : ELLM_ERR_CUDA;
}

}  // namespace ellm
