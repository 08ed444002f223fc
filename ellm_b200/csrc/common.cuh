// Shared device helpers for the attention kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ellm {

constexpr int kHeadDim = 128;            // the reference's f16 kernel hard-wires 128 as well
constexpr int kRowBytes = kHeadDim * 2;  // one K or V row in bf16
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// The reference's work partitioner (src/compiler/assign.rs:11-38): split
// [0, length) into `num` parts, the first length % num parts one longer.
// Returns false when part `id` is empty.
__host__ __device__ inline bool assign_range(long long length, long long num, long long id,
                                             long long* begin, long long* end) {
    if (length < id + 1) return false;
    long long q = length / num, r = length % num;
    if (id < r) {
        *begin = (q + 1) * id;
        *end = *begin + q + 1;
    } else {
        *begin = q * id + r;
        *end = *begin + q;
    }
    return true;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte async global->shared copy; src_bytes == 0 zero-fills the destination.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src),
                 "r"(src_bytes)
                 : "memory");
}
// The GPU's nanosecond clock: what the bounded device-side waits measure against.
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Per-CTA time stamps of the decode-step kernels, for tuning the chain of programmatic dependents
// (compiled in only with -DELLM_CHAIN_TRACE; `python -m ellm_b200.chain_trace` builds that variant
// of the library beside the product one and prints the timeline).  A kernel makes one ChainTrace at
// its start; thread 0 stamps waited() after griddepcontrol.wait, mid() / mid2() at two points of the
// kernel's choosing, and the destructor stores the record {kernel id, SM, CTA, five times}.
#ifdef ELLM_CHAIN_TRACE
constexpr unsigned kChainTraceCap = 65536;
__device__ unsigned long long g_chain_trace[kChainTraceCap * 6];
__device__ unsigned g_chain_trace_n;
struct ChainTrace {
    unsigned long long t0, t1, t2, t3;
    int kid;
    __device__ __forceinline__ explicit ChainTrace(int k) : t1(0), t2(0), t3(0), kid(k) { t0 = global_timer_ns(); }
    __device__ __forceinline__ void waited() { if (threadIdx.x == 0 && t1 == 0) t1 = global_timer_ns(); }
    __device__ __forceinline__ void mid() { if (threadIdx.x == 0 && t2 == 0) t2 = global_timer_ns(); }
    __device__ __forceinline__ void mid2() { if (threadIdx.x == 0 && t3 == 0) t3 = global_timer_ns(); }
    __device__ __forceinline__ ~ChainTrace() {
        if (threadIdx.x != 0) return;
        const unsigned long long t4 = global_timer_ns();
        const unsigned slot = atomicAdd(&g_chain_trace_n, 1u);
        if (slot >= kChainTraceCap) return;
        unsigned sm;
        asm("mov.u32 %0, %%smid;" : "=r"(sm));
        unsigned long long* r = g_chain_trace + static_cast<size_t>(slot) * 6;
        r[0] = (static_cast<unsigned long long>(kid) << 48) | (static_cast<unsigned long long>(sm) << 32) | blockIdx.x;
        r[1] = t0; r[2] = t1; r[3] = t2; r[4] = t3; r[5] = t4;
    }
};
#else
struct ChainTrace {
    __device__ __forceinline__ explicit ChainTrace(int) {}
    __device__ __forceinline__ void waited() {}
    __device__ __forceinline__ void mid() {}
    __device__ __forceinline__ void mid2() {}
};
#endif
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                            uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Transposes an 8x8 matrix of 16-bit values held across the warp (thread = row lane/4, columns
// (lane%4)*2 and +1 in one register).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}

// Byte offset of 16-byte chunk `chunk` (0..15) of row `row` in a tile of 256-byte
// rows, XOR-swizzled so that the 8 rows one ldmatrix phase touches fall in 8
// different bank groups.
__device__ __forceinline__ uint32_t swz_off(int row, int chunk) {
    return static_cast<uint32_t>(row * kRowBytes + ((chunk ^ (row & 7)) << 4));
}

// Online-softmax state of one warp over a 16-row tile: thread `lane` owns rows
// lane/4 and lane/4 + 8, and of every 8-wide column block the columns
// (lane%4)*2, +1 - the accumulator layout of m16n8k16.
struct RowState {
    float m[2];  // running max of scaled scores, log2 domain
    float l[2];  // running sum of exp2(score - m), this thread's columns only until finalised
};

// One step of the recurrence on a 16 x (8*NKB) score tile held in s[NKB][4]
// (already multiplied by scale*log2e and masked with -inf), followed by
// O += P * V for V rows [0, 8*NKB) of the swizzled smem tile at v_base.
// o[16][4]: 16 blocks of 8 head-dim columns.
template <int NKB>
__device__ __forceinline__ void softmax_pv_step(float (&s)[NKB][4], RowState& st, float (&o)[16][4],
                                                uint32_t v_base, int lane) {
    float mx[2] = {st.m[0], st.m[1]};
#pragma unroll
    for (int j = 0; j < NKB; ++j) {
        mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
        mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float corr[2], msub[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        // a row that has seen no key yet keeps m = -inf; subtract 0 there so that
        // exp2(-inf - 0) = 0 instead of exp2(-inf + inf) = NaN
        msub[r] = (mx[r] == -INFINITY) ? 0.0f : mx[r];
        corr[r] = fast_exp2(st.m[r] - msub[r]);
        st.m[r] = mx[r];
        st.l[r] *= corr[r];
    }
#pragma unroll
    for (int j = 0; j < NKB; ++j) {
        s[j][0] = fast_exp2(s[j][0] - msub[0]);
        s[j][1] = fast_exp2(s[j][1] - msub[0]);
        s[j][2] = fast_exp2(s[j][2] - msub[1]);
        s[j][3] = fast_exp2(s[j][3] - msub[1]);
        st.l[0] += s[j][0] + s[j][1];
        st.l[1] += s[j][2] + s[j][3];
    }
#pragma unroll
    for (int nb = 0; nb < 16; ++nb) {
        o[nb][0] *= corr[0];
        o[nb][1] *= corr[0];
        o[nb][2] *= corr[1];
        o[nb][3] *= corr[1];
    }
    // P (bf16) as the A operand: key blocks 2*kk and 2*kk+1 form one k16 step
    const int mat = lane >> 3, mrow = lane & 7;
#pragma unroll
    for (int kk = 0; kk < NKB / 2; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
        // ldmatrix.x4.trans: matrices (keys 0-7, d0-7), (keys 8-15, d0-7),
        // (keys 0-7, d8-15), (keys 8-15, d8-15) of this k16 step
        const int vrow = kk * 16 + (mat & 1) * 8 + mrow;
#pragma unroll
        for (int np = 0; np < 8; ++np) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(v_base + swz_off(vrow, np * 2 + (mat >> 1)), b0, b1, b2, b3);
            mma_bf16_16816(o[2 * np], a, b0, b1);
            mma_bf16_16816(o[2 * np + 1], a, b2, b3);
        }
    }
}

// S(16 x 8*NKB) = Q(16 x 128) * K^T for K rows [0, 8*NKB) of the swizzled smem tile.
// qf[8][4]: the A fragments of the 8 k16 steps over head_dim.
template <int NKB>
__device__ __forceinline__ void qk_step(const uint32_t (&qf)[8][4], uint32_t k_base, float (&s)[NKB][4],
                                        int lane) {
    const int mat = lane >> 3, mrow = lane & 7;
#pragma unroll
    for (int j = 0; j < NKB; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
    for (int jp = 0; jp < NKB / 2; ++jp) {
        // ldmatrix.x4: (keys 0-7, d0-7), (keys 0-7, d8-15), (keys 8-15, d0-7), (keys 8-15, d8-15)
        const int krow = jp * 16 + (mat >> 1) * 8 + mrow;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(k_base + swz_off(krow, ks * 2 + (mat & 1)), b0, b1, b2, b3);
            mma_bf16_16816(s[2 * jp], qf[ks], b0, b1);
            mma_bf16_16816(s[2 * jp + 1], qf[ks], b2, b3);
        }
    }
}

// ---- the decode kernel's stage, keys as the M dimension ----------------------------------
// One warp, 16 keys against up to 8 * NB query heads of one group.  With a handful of query heads
// per KV head the heads make a poor M for a 16-row MMA (half of the rows empty at 8 heads), so the
// products are taken transposed:  S^T[16 keys x 8 heads] = K . Q^T  (A = the K rows as they lie in
// shared memory, B = the query heads, register-resident) and  O^T[128 dims x 8 heads] += V^T . P^T
// (A = V read with a transposing ldmatrix, B = P^T, which is the S^T fragment turned by movmatrix).
// Per 16 keys: 8 + 8 MMAs per block of 8 heads instead of 16 + 16, half the exponentials, and O
// takes 32 registers per block of 8 heads.
// Thread layout: of every S^T / O^T fragment a thread owns heads (lane%4)*2, +1 of the block and
// keys (or dims) lane/4 and lane/4 + 8 - so the running maximum m and the sum l of a head live in
// the 8 lanes that share lane%4; l holds this thread's keys only until the piece is finalised.
template <int NB>
__device__ __forceinline__ void decode_stage_t(const uint32_t (&qb)[NB][8][2], uint32_t k_base, uint32_t v_base,
                                               long long kfirst, long long len, float scale_log2, float (&m)[NB][2],
                                               float (&l)[NB][2], float (&oT)[NB][8][4], int lane) {
    const int mat = lane >> 3, mrow = lane & 7;
    float s[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
    {
        // ldmatrix.x4: (keys 0-7, d 0-7), (keys 8-15, d 0-7), (keys 0-7, d 8-15), (keys 8-15, d 8-15) of this k16 step over head_dim
        const int krow = (mat & 1) * 8 + mrow;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t a[4];
            ldmatrix_x4(k_base + swz_off(krow, ks * 2 + (mat >> 1)), a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) mma_bf16_16816(s[nb], a, qb[nb][ks][0], qb[nb][ks][1]);
        }
    }
    const bool in_lo = kfirst + (lane >> 2) < len, in_hi = kfirst + (lane >> 2) + 8 < len;
    uint32_t pb[NB][2];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float s_lo = in_lo ? s[nb][h] * scale_log2 : -INFINITY;
            const float s_hi = in_hi ? s[nb][h + 2] * scale_log2 : -INFINITY;
            float mx = fmaxf(s_lo, s_hi);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            mx = fmaxf(mx, m[nb][h]);
            // a head that has seen no key yet keeps m = -inf; subtract 0 there so that
            // exp2(-inf - 0) = 0 instead of exp2(-inf + inf) = NaN
            const float msub = (mx == -INFINITY) ? 0.0f : mx;
            const float corr = fast_exp2(m[nb][h] - msub);
            m[nb][h] = mx;
            const float p_lo = fast_exp2(s_lo - msub), p_hi = fast_exp2(s_hi - msub);
            l[nb][h] = l[nb][h] * corr + (p_lo + p_hi);
            s[nb][h] = p_lo;
            s[nb][h + 2] = p_hi;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                oT[nb][mt][h] *= corr;
                oT[nb][mt][h + 2] *= corr;
            }
        }
        // P^T as the B operand: the two 8 x 8 blocks (keys 0-7 / 8-15 by heads) turned over
        pb[nb][0] = movmatrix_trans(pack_bf16(s[nb][0], s[nb][1]));
        pb[nb][1] = movmatrix_trans(pack_bf16(s[nb][2], s[nb][3]));
    }
    {
        // ldmatrix.x4.trans: (d 0-7, keys 0-7), (d 8-15, keys 0-7), (d 0-7, keys 8-15), (d 8-15, keys 8-15) of a 16-dim block
        const int vrow = (mat >> 1) * 8 + mrow;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            uint32_t a[4];
            ldmatrix_x4_trans(v_base + swz_off(vrow, mt * 2 + (mat & 1)), a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) mma_bf16_16816(oT[nb][mt], a, pb[nb][0], pb[nb][1]);
        }
    }
}

}  // namespace ellm
