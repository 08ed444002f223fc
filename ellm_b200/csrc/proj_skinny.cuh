// K7: the projections of a decode step - at most 16 activation rows against a whole weight
// matrix:  C[m x N] = (residual +) A[m x K] . W_nt[N x K]^T,  m <= 16.
//
// Same arithmetic as proj_tcgen05.cuh (the reference's MatMul / MatMulAdd / the GEMM part of
// MatMul3, src/compiler/mul/matmul_add.rs:128-232, src/compiler/mul/matmul3.rs:289-385), other
// regime: with so few rows every weight is used once, so the step is bound by streaming W from HBM
// (2 bytes per 2*m flops) and a 128-row tensor-memory tile would be empty.  Design for bandwidth:
//   * a CTA owns a slice of `cols` output columns (a multiple of 16) and all of K for them; the
//     grid is sized so that every CTA is resident at once (<= one per SM);
//   * the slice is brought into shared memory by 16-byte asynchronous copies, every one of them
//     requested up front (a warp instruction takes 512 contiguous bytes of one weight row).  TMA
//     was measured first and streams from DRAM at no more than ~30 GB/s per SM whatever the box
//     size (about 32 KB in flight per SM), half of what this needs; the load/store path keeps far
//     more in flight;
//   * the copies are requested before the kernel waits for its predecessor in the stream
//     (programmatic dependent launch): weights do not depend on it, activations do;
//   * then legacy warp-level MMA (m16n8k16) with the activation rows as M - the tensor core is
//     only the cheapest way to multiply up to 16 rows by a tile - the 16-wide k steps going round
//     the 8 warps; the eight partial sums of an output are added in warp order, the residual is
//     added, the sum is rounded to bf16 once;
//   * 16-column slices (the decode-step shapes) take the products transposed - the slice's columns
//     as M, the rows as one or two N blocks of 8 - and read their fragments with 16-byte
//     shared-memory loads instead of ldmatrix, which was the limit of the loop (see the product loop).
// When the activation rows leave too little shared memory for the whole slice (many rows, long K)
// the slice is taken in several passes over K.
#pragma once
#include "proj_tcgen05.cuh"
#include "rms_norm.cuh"

namespace ellm {

constexpr int kSkRows = 16;                    // activation rows = M of the MMA
constexpr int kSkWarps = 8;
constexpr int kSkThreads = kSkWarps * 32;
constexpr int kSkMaxCols = 64;                 // columns per CTA (accumulators: cols/8 x 4 registers)
constexpr int kSkSmemMax = 232448 - 4096;          // dynamic part; the kernel also has 2.2 KB of static shared memory

struct SkinnyParams {
    const __nv_bfloat16* a;
    long long lda;
    const __nv_bfloat16* w;   // [n_cols x K]
    int m_rows;               // rows of A that exist (<= 16): chunk rows x max_batch
    int batch, max_batch;     // rows with (row % max_batch) >= batch are skipped
    int k_chunks;             // K / 8: 16-byte pieces per row
    int pass_chunks;          // pieces of a weight row held in shared memory at a time (multiple of 8)
    int cols;                 // columns per CTA, multiple of 16
    int n_cols;               // N
    __nv_bfloat16* c;
    long long ldc;
    const __nv_bfloat16* residual;
    long long ldr;
    float input_norm_eps;     // >= 0: the rows of A are RMS-normalised (no weight) on their way in; < 0: taken as they are
    // ---- fused head epilogue (heads != 0): the columns are Q, K or V heads of 128, a cluster of
    // 128 / cols CTAs owns one head, and instead of storing the projection the kernel finishes it:
    // per-head RMS norm, weight, rotation at the token's position, Q to q_out, K and V into the cache
    int heads;                // 0 = plain projection; else heads of this weight matrix (n_cols / 128):
    int mat_q_heads;          //   the first mat_q_heads of them are Q heads, the next mat_k_heads K heads,
    int mat_k_heads;          //   the rest V heads (a matrix of one kind has the other counts 0)
    int q_heads;              // row pitch of q_out in heads
    __nv_bfloat16* q_out;
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    const float* q_norm_weight;   // [128] or nullptr
    const float* k_norm_weight;
    const float* rope;
    const int32_t* positions;
    long long position_index;
    long long s0, s1, s2, max_seq, rope_rows;
    float eps;
};

// shared memory: [x tile: m_rows x K bf16][128 zero bytes][slice: cols x pass_chunks x 16 bytes];
// in both tiles the 16-byte piece p of row r sits at p ^ (r & 7), so that the 8 rows one ldmatrix
// phase reads fall in 8 different bank groups.
__host__ __device__ inline int skinny_x_bytes(int k_chunks, int m_rows) { return m_rows * k_chunks * 16 + 128; }
// Largest number of pieces per pass (a multiple of 32, i.e. 512-byte runs, or all of K) that fits.
inline int skinny_pick_pass_chunks(int k_chunks, int cols, int m_rows) {
    const int room = kSkSmemMax - skinny_x_bytes(k_chunks, m_rows);
    int pc = room / (cols * 16);
    if (pc >= k_chunks) return k_chunks;
    pc &= ~31;
    return pc < 32 ? -1 : pc;   // 32 pieces per row also make room for the partial sums (512 bytes per column)
}
inline int skinny_smem_bytes(int k_chunks, int cols, int pass_chunks, int m_rows) {
    int slice = cols * pass_chunks * 16;
    if (slice < kSkWarps * kSkRows * cols * 4) slice = kSkWarps * kSkRows * cols * 4;
    return skinny_x_bytes(k_chunks, m_rows) + slice + 128;
}

// kNB16: blocks of 16 columns a CTA may own (its accumulators): 1 for the 16-column slices of the
// decode-step shapes, kSkMaxCols / 16 for anything up to kSkMaxCols columns.
// kTwo (16-column instantiation only): 9 to 16 activation rows, two N blocks of the transposed products; an
// instantiation of its own so that the code for up to 8 rows - the one-sequence decode step - stays as it is.
template <int kNB16, bool kTwo = false>
__global__ void __launch_bounds__(kSkThreads, 3) proj_skinny_kernel(const SkinnyParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int x_bytes = skinny_x_bytes(p.k_chunks, p.m_rows);
    const uint32_t x_base = smem_u32(smem), zero_addr = x_base + p.m_rows * p.k_chunks * 16, w_base = x_base + x_bytes;
    const int n0 = blockIdx.x * p.cols;
    const int passes = (p.k_chunks + p.pass_chunks - 1) / p.pass_chunks;
    ChainTrace ct(p.heads != 0 ? 7 : 8);
    // 16-column slices (the decode-step shapes) read their fragments with plain 16-byte shared-memory loads
    // instead of ldmatrix (see the product loop); both tiles are then laid out for that: the 16-byte piece
    // p of row r sits at p ^ ((r & 1) << 2).  Up to 8 activation rows are one N block of the transposed
    // products, 9 to 16 two.
    const bool few_rows = kNB16 == 1 && (kTwo || p.m_rows <= 8) && (p.k_chunks & 3) == 0 && (p.pass_chunks & 3) == 0;
    constexpr bool two_blocks = kTwo;

    // pieces [pass * pass_chunks, ...) of every row of the slice; rows past N arrive as zeros
    auto request_pass = [&](int pass) {
        const int c_begin = pass * p.pass_chunks;
        const int pc = min(p.pass_chunks, p.k_chunks - c_begin);
        // row by row, the whole CTA on one row at a time (4 KB contiguous per sweep streams better from
        // DRAM than eight rows at once); no index division
        for (int n = 0; n < p.cols; ++n) {
            const bool real = n0 + n < p.n_cols;
            const __nv_bfloat16* src = p.w + (real ? (static_cast<long long>(n0 + n) * p.k_chunks + c_begin) * 8 : 0);
            const uint32_t dst = w_base + n * p.pass_chunks * 16;
            const int sw = few_rows ? (n & 1) << 2 : n & 7;
            for (int cc = threadIdx.x; cc < pc; cc += kSkThreads)
                cp_async_16(dst + ((cc ^ sw) << 4), src + (real ? cc * 8 : 0), real ? 16 : 0);
        }
        cp_async_commit();
    };
    request_pass(0);
    // fused head epilogue: a CTA's shared memory may be written by its cluster peers only once it runs;
    // every CTA says so here and checks the others just before the exchange
    if (p.heads != 0) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    // activations (and the residual) are the previous kernels' output: wait for them
    asm volatile("griddepcontrol.wait;" ::: "memory");
    ct.waited();
    // only now may the next kernel of the stream start its own prologue: whatever it reads before
    // its own wait (a decode kernel with early streaming: the positions, older cache rows) is then
    // older than everything this kernel waited for
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // fused head epilogue: what its last step needs from global memory - the token's position, its
    // rotation row, the norm weights - is requested now, two dependent round trips ahead of its use
    long long ep_pos = -1;
    float4 ep_wv = make_float4(1.f, 1.f, 1.f, 1.f), ep_cs = make_float4(1.f, 0.f, 1.f, 0.f);
    if (p.heads != 0 && threadIdx.x < 4 * p.m_rows) {
        const int m = threadIdx.x >> 2, quad = threadIdx.x & 3, b = m % p.max_batch;
        if (b < p.batch) {
            ep_pos = (p.positions ? static_cast<long long>(p.positions[b]) : p.position_index) + m / p.max_batch;
            const int head = n0 >> 7, ch = (n0 & 127) + quad * 4;
            const int kind = head >= p.mat_q_heads + p.mat_k_heads ? 2 : (head >= p.mat_q_heads ? 1 : 0);
            if (kind != 2 && ep_pos >= 0 && ep_pos < p.rope_rows) {
                const float* wgt = kind == 0 ? p.q_norm_weight : p.k_norm_weight;
                if (wgt) ep_wv = *reinterpret_cast<const float4*>(wgt + ch);
                ep_cs = *reinterpret_cast<const float4*>(p.rope + ep_pos * kHeadDim + ch);  // cos0 sin0 cos1 sin1
            }
        }
    }
    if (p.input_norm_eps >= 0.0f) {
        // the layer's input norm, y = x / (sqrt(mean x^2) + eps) rounded to bf16, on the few rows
        // of a decode step (src/kernel/generic/rms_norm.rs:6-26); the same code as rms_norm_kernel
        __shared__ float warp_sums[8];
        __shared__ float s_rrms;
        for (int m = 0; m < p.m_rows; ++m) {
            const bool live = (m % p.max_batch) < p.batch;   // uniform over the CTA
            const uint4* src = reinterpret_cast<const uint4*>(p.a + (live ? m * p.lda : 0));
            const float rrms = live ? block_row_rrms(src, p.k_chunks, p.k_chunks * 8, p.input_norm_eps, warp_sums, &s_rrms) : 0.0f;
            for (int c = threadIdx.x; c < p.k_chunks; c += kSkThreads)
                *reinterpret_cast<uint4*>(smem + (m * p.k_chunks + (c ^ (few_rows ? (m & 1) << 2 : m & 7))) * 16) =
                    live ? scale_piece(src[c], rrms) : make_uint4(0u, 0u, 0u, 0u);
        }
    } else {
        for (int m = 0; m < p.m_rows; ++m) {
            const bool live = (m % p.max_batch) < p.batch;
            const __nv_bfloat16* src = p.a + (live ? m * p.lda : 0);
            for (int c = threadIdx.x; c < p.k_chunks; c += kSkThreads)
                cp_async_16(x_base + (m * p.k_chunks + (c ^ (few_rows ? (m & 1) << 2 : m & 7))) * 16, src + c * 8, live ? 16 : 0);
        }
    }
    if (threadIdx.x < 8) cp_async_16(zero_addr + threadIdx.x * 16, p.a, 0);   // 128 zero bytes: what every missing row reads
    cp_async_commit();
    // the residual values of this thread's outputs, requested now, used at the very end
    const int outs = p.m_rows * p.cols;
    float res[4] = {0.f, 0.f, 0.f, 0.f};
    if (p.residual) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + i * kSkThreads;
            const int m = idx / p.cols, n = n0 + idx % p.cols;
            if (idx < outs && (m % p.max_batch) < p.batch && n < p.n_cols) res[i] = __bfloat162float(p.residual[m * p.ldr + n]);
        }
    }

    // (16-column slices, at most 8 rows: four accumulators of the transposed products, see below)
    float tacc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) tacc[i][0] = tacc[i][1] = tacc[i][2] = tacc[i][3] = 0.0f;
    float acc[kNB16 * 2][4];
#pragma unroll
    for (int i = 0; i < kNB16 * 2; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
    const int nblocks16 = p.cols >> 4;
    const int a_row = lane & 15;
    const bool a_live = a_row < p.m_rows;
    for (int pass = 0; pass < passes; ++pass) {
        if (pass > 0) {
            __syncthreads();   // every warp is done with the previous part of the slice
            request_pass(pass);
        }
        cp_async_wait<0>();
        __syncthreads();
        ct.mid();   // (trace) slice and rows are in shared memory
        const int c_begin = pass * p.pass_chunks;
        const int steps = min(p.pass_chunks, p.k_chunks - c_begin) >> 1;   // 16-wide k steps of this pass
        if (few_rows) {
            // 16 columns: the products are taken transposed - the slice's 16
            // columns are the M side of m16n8k16, the rows the N side, one product per 16 k instead of
            // two - and the fragments come from plain 16-byte shared-memory loads: ldmatrix delivers
            // one 8x8 matrix per ~3 clocks per SM here (measured: the slice's 128 KB took 2.4 us through
            // it, whatever the products did), a 16-byte load per lane four times that.  A lane's 16 bytes
            // of a row are 4 k-pairs; which k a fragment register stands for is free as long as the
            // slice and the rows agree, so lane (g, t) reads piece 4 * kb + t of slice rows g and g + 8
            // and of activation row g, and feeds register pairs 0,1 to one product and 2,3 to the next.
            // A quarter-warp then touches 8 different pieces (rows g, g + 1 sit in opposite halves of
            // a 128-byte bank line): no conflicts.  Four independent accumulators, added at the end.
            const int g = lane >> 2, t = lane & 3, sw = (g & 1) << 2;
            const int kblocks = steps >> 1;   // 32-k blocks of this pass
            const uint32_t w_lo = w_base + g * p.pass_chunks * 16, w_hi = w_lo + 8 * p.pass_chunks * 16;
            const bool x_live = g < p.m_rows;
            const uint32_t x_row = x_base + g * p.k_chunks * 16;
            if (two_blocks) {
                // 9 to 16 rows: rows g and g + 8 are two N blocks against the same slice fragments; accumulators
                // 0, 1 belong to rows 0-7 and 2, 3 to rows 8-15
                const bool x_live_hi = g + 8 < p.m_rows;
                const uint32_t x_row_hi = x_row + 8 * p.k_chunks * 16;
                for (int kb = warp; kb < kblocks; kb += kSkWarps) {
                    const int c = kb * 4 + t;
                    const uint4 lo = lds128(w_lo + ((c ^ sw) << 4)), hi = lds128(w_hi + ((c ^ sw) << 4));
                    const uint32_t x_off = ((c_begin + c) ^ sw) << 4, z_off = (((c_begin + c) ^ sw) & 7) << 4;
                    const uint4 x0 = lds128(x_live ? x_row + x_off : zero_addr + z_off);
                    const uint4 x1 = lds128(x_live_hi ? x_row_hi + x_off : zero_addr + z_off);
                    const uint32_t a0[4] = {lo.x, hi.x, lo.y, hi.y}, a1[4] = {lo.z, hi.z, lo.w, hi.w};
                    mma_bf16_16816(tacc[0], a0, x0.x, x0.y);
                    mma_bf16_16816(tacc[1], a1, x0.z, x0.w);
                    mma_bf16_16816(tacc[2], a0, x1.x, x1.y);
                    mma_bf16_16816(tacc[3], a1, x1.z, x1.w);
                }
                continue;
            }
            for (int kb = warp; kb < kblocks; kb += 2 * kSkWarps) {
                uint4 lo[2], hi[2], xr[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int c = (kb + u * kSkWarps) * 4 + t;
                    if (kb + u * kSkWarps < kblocks) {
                        lo[u] = lds128(w_lo + ((c ^ sw) << 4));
                        hi[u] = lds128(w_hi + ((c ^ sw) << 4));
                        xr[u] = lds128(x_live ? x_row + (((c_begin + c) ^ sw) << 4) : zero_addr + ((((c_begin + c) ^ sw) & 7) << 4));
                    }
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    if (kb + u * kSkWarps < kblocks) {
                        const uint32_t a0[4] = {lo[u].x, hi[u].x, lo[u].y, hi[u].y}, a1[4] = {lo[u].z, hi[u].z, lo[u].w, hi[u].w};
                        mma_bf16_16816(tacc[2 * u], a0, xr[u].x, xr[u].y);
                        mma_bf16_16816(tacc[2 * u + 1], a1, xr[u].z, xr[u].w);
                    }
                }
            }
            continue;
        }
        for (int step = warp; step < steps; step += kSkWarps) {
            uint32_t af[4];
            {
                const int piece = c_begin + step * 2 + (lane >> 4);
                const uint32_t addr = a_live ? x_base + (a_row * p.k_chunks + (piece ^ (a_row & 7))) * 16 : zero_addr;
                ldmatrix_x4(addr, af[0], af[1], af[2], af[3]);
            }
#pragma unroll
            for (int nb = 0; nb < kNB16; ++nb) {
                if (nb < nblocks16) {
                    // matrices: (cols 0-7, k 0-7), (cols 0-7, k 8-15), (cols 8-15, k 0-7), (cols 8-15, k 8-15)
                    const int n = nb * 16 + ((lane >> 4) << 3) + (lane & 7), piece = step * 2 + ((lane >> 3) & 1);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(w_base + (n * p.pass_chunks + (piece ^ (n & 7))) * 16, b0, b1, b2, b3);
                    mma_bf16_16816(acc[nb * 2], af, b0, b1);
                    mma_bf16_16816(acc[nb * 2 + 1], af, b2, b3);
                }
            }
        }
    }
    // every warp is done with the slice: the partial sums go over it
    __syncthreads();
    ct.mid2();  // (trace) the product loop is done
    float* part = reinterpret_cast<float*>(smem + x_bytes);   // [warp][row][col]
    if (few_rows) {
        // transposed accumulators: this lane holds columns lane/4 and lane/4 + 8 of rows (lane%4)*2, +1
        const int col = lane >> 2, m0 = (lane & 3) * 2;
        float* dst = part + (warp * kSkRows + m0) * p.cols + col;
        if (two_blocks) {
            float* dst_hi = dst + 8 * p.cols;   // rows 8-15
            dst[0] = tacc[0][0] + tacc[1][0];
            dst[p.cols] = tacc[0][1] + tacc[1][1];
            dst[8] = tacc[0][2] + tacc[1][2];
            dst[p.cols + 8] = tacc[0][3] + tacc[1][3];
            dst_hi[0] = tacc[2][0] + tacc[3][0];
            dst_hi[p.cols] = tacc[2][1] + tacc[3][1];
            dst_hi[8] = tacc[2][2] + tacc[3][2];
            dst_hi[p.cols + 8] = tacc[2][3] + tacc[3][3];
        } else {
            dst[0] = (tacc[0][0] + tacc[1][0]) + (tacc[2][0] + tacc[3][0]);
            dst[p.cols] = (tacc[0][1] + tacc[1][1]) + (tacc[2][1] + tacc[3][1]);
            dst[8] = (tacc[0][2] + tacc[1][2]) + (tacc[2][2] + tacc[3][2]);
            dst[p.cols + 8] = (tacc[0][3] + tacc[1][3]) + (tacc[2][3] + tacc[3][3]);
        }
    } else {
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
        for (int i = 0; i < kNB16 * 2; ++i) {
            if (i * 8 < p.cols) {
                float* dst = part + (warp * kSkRows) * p.cols + i * 8 + c0;
                dst[r0 * p.cols] = acc[i][0];
                dst[r0 * p.cols + 1] = acc[i][1];
                dst[(r0 + 8) * p.cols] = acc[i][2];
                dst[(r0 + 8) * p.cols + 1] = acc[i][3];
            }
        }
    }
    __syncthreads();
    if (p.heads != 0) {
        // ---- fused head epilogue.  Thread t < 4 * m_rows owns 4 consecutive channels of one row of this
        // CTA's 16 columns: exactly what one lane of qk_norm_rope_append_kernel owns, and the arithmetic
        // below is that kernel's, so that both routes give the same bits.
        __shared__ float ss_all[32][kSkRows];   // the head's 32 four-channel sums of squares of every row
        const int t = threadIdx.x, m = t >> 2, quad = t & 3;
        const bool mine = t < 4 * p.m_rows;
        const bool live = mine && (m % p.max_batch) < p.batch;
        const uint32_t crank = cluster_ctarank();          // which 16 columns of the head
        int head = n0 >> 7, kind = 0;                       // head of this matrix -> kind and head of that kind
        if (head >= p.mat_q_heads + p.mat_k_heads) { kind = 2; head -= p.mat_q_heads + p.mat_k_heads; }
        else if (head >= p.mat_q_heads) { kind = 1; head -= p.mat_q_heads; }
        float x[4] = {0.f, 0.f, 0.f, 0.f};
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // every CTA of the head has started
        if (mine) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float sum = 0.0f;
#pragma unroll
                for (int w = 0; w < kSkWarps; ++w) sum += part[(w * kSkRows + m) * p.cols + quad * 4 + e];
                x[e] = bf16_round(sum);   // the projection as it would have been stored
            }
            if (kind != 2) {
                const float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
                const uint32_t mine_addr = smem_u32(&ss_all[crank * 4 + quad][m]);
#pragma unroll
                for (uint32_t peer = 0; peer < 8; ++peer)
                    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(mapa_shared(mine_addr, peer)), "f"(ss) : "memory");
            }
        }
        cluster_sync_all();   // every CTA of the head has every partial sum
        if (live) {
            const int b = m % p.max_batch;
            const long long pos = ep_pos;
            const int ch = (n0 & 127) + quad * 4;   // channel of x[0] inside the head
            if (kind == 2) {
                if (pos >= 0 && pos < p.max_seq && pos < p.rope_rows) {   // as K: no rotation row, no cache write
                    uint2 v;
                    v.x = pack_bf16(x[0], x[1]);
                    v.y = pack_bf16(x[2], x[3]);
                    *reinterpret_cast<uint2*>(p.v_cache + b * p.s0 + head * p.s1 + pos * p.s2 + ch) = v;
                }
            } else if (!(kind == 1 && pos >= p.max_seq) && pos >= 0 && pos < p.rope_rows) {
                // the butterfly of the separate kernel: lane i adds lane i ^ 16, then ^ 8, 4, 2, 1
                float tsum[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) tsum[i] = ss_all[i][m];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    float nxt[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) nxt[i] = tsum[i] + tsum[i ^ o];
#pragma unroll
                    for (int i = 0; i < 32; ++i) tsum[i] = nxt[i];
                }
                const float rrms = 1.0f / (sqrtf(tsum[0] / static_cast<float>(kHeadDim)) + p.eps);
                const float4 wv = ep_wv, cs = ep_cs;
                const float y0 = x[0] * rrms * wv.x, y1 = x[1] * rrms * wv.y, y2 = x[2] * rrms * wv.z, y3 = x[3] * rrms * wv.w;
                uint2 outv;
                outv.x = pack_bf16(y0 * cs.x - y1 * cs.y, y0 * cs.y + y1 * cs.x);
                outv.y = pack_bf16(y2 * cs.z - y3 * cs.w, y2 * cs.w + y3 * cs.z);
                __nv_bfloat16* dst = kind == 0 ? p.q_out + (static_cast<long long>(m) * p.q_heads + head) * kHeadDim
                                                      : p.k_cache + b * p.s0 + head * p.s1 + pos * p.s2;
                *reinterpret_cast<uint2*>(dst + ch) = outv;
            }
        }
        return;   // all remote stores into this CTA's shared memory were before the cluster barrier
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = threadIdx.x + i * kSkThreads;
        if (idx >= outs) break;
        const int m = idx / p.cols, j = idx % p.cols, n = n0 + j;
        if ((m % p.max_batch) >= p.batch || n >= p.n_cols) continue;
        float sum = 0.0f;
#pragma unroll
        for (int w = 0; w < kSkWarps; ++w) sum += part[(w * kSkRows + m) * p.cols + j];
        p.c[m * p.ldc + n] = __float2bfloat16_rn(sum + res[i]);
    }
}

}  // namespace ellm
