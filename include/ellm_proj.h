/* C ABI of the projections either side of the attention operator, on the B200 tensor cores.
 *
 * These are the reference's callers of the attention path (its operators MatMul3 and MatMulAdd),
 * kept behind the same shape of interface: a constructor that binds the buffers once and a
 * run(position_index, position_interval, batch_size, cpu_num, thread_id) that every worker thread
 * of the executor calls (src/compiler/operator.rs:68-75); thread_id 0 launches, the others return
 * ELLM_OK at once.  Status codes, ellm_last_error() and the stream / async convention are those of
 * ellm_attn.h.  All matrices are bf16, row-major, 16-byte aligned; weights are N x K ("W_nt", as
 * the reference stores them, src/compiler/mul/matmul3.rs:22-28); accumulation is fp32.
 *
 * Rows: activations are [chunk row r][sequence b of max_batch] like the attention operator's q and
 * out, so matrix row m = r * max_batch + b.  A run covers chunk rows [0, position_interval) and
 * sequences [0, batch_size); rows of the other sequences are neither computed into outputs nor
 * written.  (The reference passes its row count in batch_size and has no chunk dimension here:
 * matmul3.rs:289-303; with position_interval = 1 and max_batch = its m_row the two agree.)
 */
#ifndef ELLM_PROJ_H
#define ELLM_PROJ_H

#include <stddef.h>
#include <stdint.h>

#include "ellm_attn.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- MatMul3: Q, K, V projections + per-head RMSNorm + RoPE + KV-cache write ------------------
 * Replaces MatMul3::new / MatMul3::run (src/compiler/mul/matmul3.rs:60-119, 289-385) with its
 * finalize step on every finished 128-wide head of Q and K (matmul3.rs:230-262: rms_norm then
 * complex_mul; y = x / (sqrt(mean x^2) + eps), src/kernel/generic/rms_norm.rs:6-26; interleaved
 * pairs times (cos, sin), src/kernel/generic/complex_mul.rs:3-20), and the write of K and V into
 * the static cache that the reference plans as output_to_kv (src/compiler/zip_map/
 * complex_zip.rs:92-98).  Differences, on purpose: the rotation row is the one of the token's
 * position (the reference's finalize always reads row 0 of the table, matmul3.rs:251); optional
 * per-channel norm weights multiply the normalised head before the rotation (the reference's norm
 * has none); the projected row is rounded to bf16 before the norm, exactly as if it had been stored
 * and read back, so this entry point and ellm_qk_norm_rope_append after a plain projection give
 * the same bits. */
typedef struct ellm_matmul3 ellm_matmul3;

typedef struct ellm_matmul3_desc {
    const void* hidden;        /* hidden_ptr: A [m_row x col]                                   */
    size_t hidden_row_stride;  /* elements between rows of A; 0 = col                           */
    const void* wq_nt;         /* q_weight_ptr_nt [b_q_row x col]                               */
    const void* wk_nt;         /* k_weight_ptr_nt [b_kv_row x col]                              */
    const void* wv_nt;         /* v_weight_ptr_nt [b_kv_row x col]                              */
    void* q_state;             /* q_state_ptr [m_row x b_q_row] = [rows, max_batch, q_heads, 128] */
    void* k_cache;             /* K rows go here at (b, kv head, position) ...                  */
    void* v_cache;             /* ... and V rows here, instead of k_state_ptr / v_state_ptr     */
    size_t kv_strides[4];      /* as in ellm_attn_desc                                          */
    const float* rope;         /* rope_ptr: [rope_rows x 128] fp32, (cos, sin) interleaved      */
    size_t rope_rows;
    const float* q_norm_weight; /* [128] fp32 or NULL                                           */
    const float* k_norm_weight; /* [128] fp32 or NULL                                           */
    size_t head_dim;           /* 128                                                           */
    size_t m_row;              /* most rows a run is given = max_interval * max_batch           */
    size_t col;                /* K, a multiple of 64                                           */
    size_t b_q_row;            /* Nq  = q_heads * 128                                           */
    size_t b_kv_row;           /* Nkv = kv_heads * 128                                          */
    size_t max_batch;
    size_t max_seq;
    float eps;
    int device;
    void* stream;
    int async;                 /* 0: run() returns after the stream drained; 1: only enqueues   */
    /* Optional: the layer's input norm taken into the operator.  With input_norm != 0, `hidden` is
     * the layer's un-normalised input and every row is first replaced by x / (sqrt(mean x^2) +
     * input_norm_eps), rounded to bf16 - the weight-free rms_norm the reference runs as its own
     * operator before this one (src/qwen3_moe/decoder_layer.rs:139-143, src/kernel/generic/
     * rms_norm.rs:6-26); same bits as ellm_rms_norm followed by this operator.  A decode step
     * normalises its few rows inside the projection kernel; a chunk writes the normalised rows to
     * normed_scratch ([m_row x col] bf16, the caller's, may be shared by all layers) first. */
    int input_norm;
    float input_norm_eps;
    void* normed_scratch;
} ellm_matmul3_desc;

int ellm_matmul3_create(const ellm_matmul3_desc* desc, ellm_matmul3** out);
int ellm_matmul3_destroy(ellm_matmul3* h);
/* Chunk row r of sequence b is the token at position position_index + r. */
int ellm_matmul3_run(ellm_matmul3* h, size_t position_index, size_t position_interval, size_t batch_size,
                     size_t cpu_num, size_t thread_id);
/* Extension: sequence b starts its chunk at positions[b] (device int32[batch_size]). */
int ellm_matmul3_run_ragged(ellm_matmul3* h, const int32_t* positions, size_t position_interval,
                            size_t batch_size, size_t cpu_num, size_t thread_id);

/* Decode steps (at most 16 rows) run one kernel per weight matrix that projects and finishes the
 * heads (default), or - with on = 0 - the projection kernel followed by ellm_qk_norm_rope_append's
 * kernel; both give the same bits.  A tuning / comparison knob. */
int ellm_matmul3_set_decode_fusion(ellm_matmul3* h, int on);

/* ---- MatMulAdd: output = residual + A . W_nt^T ------------------------------------------------
 * Replaces MatMulAdd::new / run (src/compiler/mul/matmul_add.rs:60-126, 128-232: C = residual,
 * then C += A x B); with residual NULL it is the plain MatMul (src/compiler/mul/matmul.rs).
 * The sum is formed in fp32 and rounded to bf16 once.  output may alias residual. */
typedef struct ellm_matmul_add ellm_matmul_add;

typedef struct ellm_matmul_add_desc {
    const void* a;             /* ptr1: A [m_max x k_max]                                       */
    size_t a_row_stride;       /* elements; 0 = k_max                                           */
    const void* w_nt;          /* ptr2: [n_max x k_max]                                         */
    const void* residual;      /* ptr3: [m_max x n_max] or NULL                                 */
    size_t residual_row_stride; /* elements; 0 = n_max                                          */
    void* output;              /* output_ptr: [m_max x n_max]                                   */
    size_t output_row_stride;  /* elements; 0 = n_max                                           */
    size_t m_max;              /* max_interval * max_batch                                      */
    size_t n_max;              /* a multiple of 8                                               */
    size_t k_max;              /* a multiple of 64                                              */
    size_t max_batch;
    int device;
    void* stream;
    int async;
} ellm_matmul_add_desc;

int ellm_matmul_add_create(const ellm_matmul_add_desc* desc, ellm_matmul_add** out);
int ellm_matmul_add_destroy(ellm_matmul_add* h);
int ellm_matmul_add_run(ellm_matmul_add* h, size_t position_index, size_t position_interval, size_t batch_size,
                        size_t cpu_num, size_t thread_id);

/* Launches and device time of a handle's kernel since profiling was switched on (events around
 * every launch; for measurement only).  `which`: 0 = ellm_matmul3, 1 = ellm_matmul_add. */
int ellm_matmul_set_profiling(void* handle, int which, int on);
int ellm_matmul_kernel_stats(void* handle, int which, uint64_t* launches, uint64_t* timed_launches, double* ms);
/* Waits for the handle's stream and reports a device-side wait that ran out since the last check
 * (ELLM_ERR_DEVICE_TIMEOUT).  Synchronous handles check after every run; enqueue-only handles
 * (async = 1) add nothing to the stream and are checked here. */
int ellm_matmul_check(void* handle, int which);
/* Bound of every device-side wait of the handle's kernel, nanoseconds (default 2e9). */
int ellm_matmul_set_wait_timeout(void* handle, int which, unsigned long long ns);
/* Tuning knob of the tensor-memory kernel: two CTAs of a cluster share a 256 x 256 tile
 * (tcgen05 cta_group::2; each CTA loads its 128 rows of A and half of the weight tile).
 * mode -1 (default): when every pair gets at least two tiles; 0: never; 1: whenever rows > 128. */
int ellm_matmul_set_pairing(void* handle, int which, int mode);
/* Test hook for the failure path: the tensor-memory kernel's loader leaves operand block `item`
 * (counted over the first CTA's k-blocks) unloaded, so the wait on it runs out after the bound above
 * and the run reports ELLM_ERR_DEVICE_TIMEOUT; -1 switches it off. */
int ellm_matmul_debug_skip_load(void* handle, int which, int item);

#ifdef __cplusplus
}
#endif
#endif
