/* C ABI of the B200 attention path for eLLM.
 *
 * This library stands in for ONE operator of the reference crate: the attention
 * node of its static graph.  Every entry point names the reference interface it
 * replaces (paths relative to the reference project root).  Signatures carry
 * plain pointers and sizes only.  All data pointers are DEVICE pointers unless a
 * parameter is named *_host.  Every function returns an ellm_status; nothing
 * aborts the process (the reference panics instead: Cargo.toml `panic = "abort"`).
 *
 * Element type: bf16 in, bf16 out, fp32 accumulation, fp32 log-sum-exp.
 */
#ifndef ELLM_ATTN_H
#define ELLM_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ellm_status {
    ELLM_OK = 0,
    ELLM_ERR_INVALID_ARG = 1,   /* null pointer, bad head counts, misaligned base, position past max_seq */
    ELLM_ERR_CUDA = 2,          /* a CUDA runtime / driver call failed; see ellm_last_error() */
    ELLM_ERR_DEVICE_TIMEOUT = 3,/* a bounded device-side wait ran out; results of that call are invalid */
    ELLM_ERR_UNSUPPORTED = 4,   /* shape outside what the kernels implement (e.g. head_size != 128) */
    ELLM_ERR_NO_MEMORY = 5
} ellm_status;

typedef enum ellm_dtype { ELLM_DTYPE_BF16 = 0 } ellm_dtype;

/* Which kernel ellm_attn_run picks for a chunk of more than one row. */
typedef enum ellm_prefill_kernel {
    ELLM_PREFILL_AUTO = 0,     /* tcgen05 kernel from 16 packed rows (chunk rows x query heads per KV head) up,
                                  else the warp-MMA kernel */
    ELLM_PREFILL_TCGEN05 = 1,
    ELLM_PREFILL_WARP_MMA = 2
} ellm_prefill_kernel;

typedef struct ellm_attn ellm_attn;

/* The arguments of Attention::new (src/compiler/mul/attention.rs:41-67) as
 * Tensor::attention passes them (src/ptensor/tensor.rs:107-139), plus what a
 * device needs that a CPU does not.
 *
 * Layouts (elements, not bytes):
 *   q, out : [chunk rows, max_batch, q_heads, head_size] row-major - the
 *            reference addresses both with the MAX batch stride
 *            (attention.rs:86,118-119).
 *   k_cache, v_cache : element (b, kvh, pos, c) at
 *            b*kv_strides[0] + kvh*kv_strides[1] + pos*kv_strides[2] + c*kv_strides[3],
 *            the stride vector the reference takes from the permuted K tensor
 *            (src/qwen3_moe/attention.rs:149-166).  kv_strides[3] must be 1;
 *            the others must be multiples of 8 elements (16 bytes).
 *   lse    : [chunk rows, max_batch, q_heads] fp32, natural log, softmax scale
 *            included; may be NULL.  The reference drops it.
 *   k_new, v_new : [chunk rows, max_batch, kv_heads, head_size]; the chunk's new
 *            K/V rows which run() first writes into the cache at
 *            [position_index, position_index+interval) - the reference's
 *            output_to_kv intent (src/compiler/zip_map/complex_zip.rs:92-98).
 *            Both NULL = the caller already wrote the cache.
 * A query head h reads KV head h / (q_heads / kv_heads).
 */
typedef struct ellm_attn_desc {
    const void* q;
    void* k_cache;
    void* v_cache;
    void* out;
    float* lse;
    const void* k_new;
    const void* v_new;
    size_t max_batch;      /* Attention::new batch_size: the allocated batch */
    size_t q_heads;        /* attention_head_num */
    size_t kv_heads;       /* kv_head_num */
    size_t head_size;      /* 128 */
    size_t kv_strides[4];
    size_t max_seq;        /* rows per (sequence, kv head) the cache holds */
    size_t max_interval;   /* most chunk rows one run() will be given (sizes q/out) */
    float scale;           /* inverse_sqrt_head */
    int dtype;             /* ellm_dtype */
    int device;            /* CUDA device ordinal */
    void* stream;          /* cudaStream_t the kernels are enqueued on; NULL = legacy default stream */
    int async;             /* 0: run() returns after the stream has drained (what the
                              executor's barrier expects, src/serving/start.rs:69-73);
                              1: run() only enqueues */
    int prefill_kernel;    /* ellm_prefill_kernel */
} ellm_attn_desc;

/* Attention::new.  Allocates the handle's split-KV workspace on desc->device. */
int ellm_attn_create(const ellm_attn_desc* desc, ellm_attn** out);
int ellm_attn_destroy(ellm_attn* h);

/* Attention::run(position_index, position_interval, batch_size, cpu_num,
 * thread_id) (src/compiler/mul/attention.rs:69-76; same signature as every
 * Operator::run, src/compiler/operator.rs:68-75).  Chunk row r of sequence b is
 * the token at absolute position position_index + r and attends keys
 * 0..=position_index + r.  The executor calls this from every worker thread;
 * thread_id 0 launches, every other thread_id returns ELLM_OK at once and the
 * executor's barrier does the rest. */
int ellm_attn_run(ellm_attn* h, size_t position_index, size_t position_interval,
                  size_t batch_size, size_t cpu_num, size_t thread_id);

/* Extension (the reference has one position for the whole batch): sequence b
 * starts its chunk at positions[b] (device int32[batch_size]). */
int ellm_attn_run_ragged(ellm_attn* h, const int32_t* positions, size_t position_interval,
                         size_t batch_size, size_t cpu_num, size_t thread_id);

/* Same step for a caller whose activations live in HOST memory (the reference's
 * buffers are host allocations, src/memory/allocator.rs:4-27): copies q (and
 * k_new/v_new, positions when non-NULL) to the handle's bound device buffers,
 * runs, copies out (and lse) back, and returns when the results are in host
 * memory.  The KV cache stays resident on the device.  Decode steps with positions_host and
 * page-locked buffers are captured once into a CUDA graph and replayed for as long as the same
 * buffers are passed; in that graph one small kernel fetches all inputs from the host buffers
 * and the last kernel of the step stores O and LSE directly into out_host / lse_host, so the
 * handle's device out / lse buffers are not written by such a step.  Calls on one handle must
 * not overlap. */
int ellm_attn_run_host(ellm_attn* h, const void* q_host, const void* k_new_host,
                       const void* v_new_host, void* out_host, float* lse_host,
                       const int32_t* positions_host, size_t position_index,
                       size_t position_interval, size_t batch_size);

/* allocate_init (src/memory/allocator.rs:16-27) for device memory: zero-filled,
 * 256-byte aligned.  Unlike the reference, which never frees, there is a free. */
int ellm_device_alloc(int device, size_t bytes, void** out);
int ellm_device_free(int device, void* ptr);

/* The static, non-paged KV cache as one object: K and V as [layer, sequence, kv_head,
 * position, head_size] bf16 in device memory, allocated once at their maximum shape, zero-
 * filled and never resized - the reference's max-shape, never-freed K/V buffers
 * (src/memory/allocator.rs:16-27; one private buffer per layer by name,
 * src/memory/cache.rs:69-75).  ellm_kv_cache_layer hands out a layer's K and V base pointers and
 * the stride vector an ellm_attn_desc takes (sequence, kv_head, position, head_size - a KV
 * head's rows are contiguous 256-byte lines).  Any of k, v, kv_strides may be NULL. */
typedef struct ellm_kv_cache ellm_kv_cache;
int ellm_kv_cache_create(int device, size_t layers, size_t max_batch, size_t kv_heads,
                         size_t max_seq, size_t head_size, ellm_kv_cache** out);
int ellm_kv_cache_destroy(ellm_kv_cache* cache);
int ellm_kv_cache_layer(const ellm_kv_cache* cache, size_t layer, void** k, void** v,
                        size_t kv_strides[4]);

/* The KV-append step alone (complex_zip.rs:92-98 semantics): rows
 * src[(r*max_batch + b)*kv_heads + kvh][head_size] -> cache row
 * (b, kvh, position_b + r).  positions NULL = position_index for every b. */
int ellm_kv_append(void* cache, const void* src, const size_t kv_strides[4], size_t max_batch,
                   size_t kv_heads, size_t head_size, size_t max_seq, size_t position_index,
                   const int32_t* positions, size_t position_interval, size_t batch_size,
                   int device, void* stream);

/* The step between the QKV projection and attention, fused: per-head RMSNorm
 * (y = x / (sqrt(mean x^2) + eps), src/kernel/generic/rms_norm.rs:6-26), interleaved RoPE
 * (src/kernel/generic/complex_mul.rs:3-20) on every Q and K head - the reference's
 * matmul_finalize_rmsnorm_rope_inplace_3x128, src/kernel/x86_64/f16_512/
 * matmul_rms_complex.rs:76-96 - and the write of K and V into the cache at the chunk's
 * positions (output_to_kv, src/compiler/zip_map/complex_zip.rs:92-98).
 * q_in/q_out [rows, max_batch, q_heads, 128] (may alias), k_in/v_in [rows, max_batch, kv_heads,
 * 128], bf16; q_in_row_stride / kv_in_row_stride (elements, 0 = contiguous) let the three inputs be
 * column blocks of one fused projection output; q_weight/k_weight fp32[128] or NULL (the
 * reference's norm has no weight);
 * rope fp32 [rope_rows, 128] of interleaved (cos, sin), row = absolute position
 * (src/qwen3_moe/rope.rs:7-28); positions as in ellm_attn_run_ragged or NULL. */
int ellm_qk_norm_rope_append(const void* q_in, const void* k_in, const void* v_in, void* q_out,
                             void* k_cache, void* v_cache, const float* q_weight,
                             const float* k_weight, const float* rope, size_t rope_rows,
                             const size_t kv_strides[4], size_t max_batch, size_t q_heads,
                             size_t kv_heads, size_t head_size, size_t max_seq,
                             size_t position_index, const int32_t* positions,
                             size_t position_interval, size_t batch_size, float eps,
                             size_t q_in_row_stride, size_t kv_in_row_stride, int device,
                             void* stream);

/* Row-wise weight-free RMS normalisation y = x / (sqrt(mean x^2) + eps) of a [rows, length] bf16
 * matrix (length a multiple of 8): the reference's rms_norm, src/kernel/generic/rms_norm.rs:6-26,
 * the input norm that produces what the QKV projection reads
 * (src/qwen3_moe/decoder_layer.rs:139-143).  x and y may alias. */
int ellm_rms_norm(const void* x, void* y, size_t rows, size_t length, float eps, int device,
                  void* stream);

/* Combine `parts` partial results of the same query rows taken over disjoint key
 * sets: L = log sum_i exp(L_i), O = sum_i O_i exp(L_i - L).  No counterpart in the
 * reference (it never splits the key range); it is the exchange step of the
 * split-KV decode and of sequence-chunk sharding across GPUs.
 * o_parts [parts, rows, head_size] fp32, lse_parts [parts, rows] fp32,
 * out [rows, head_size] bf16, lse_out [rows] fp32 (may be NULL). */
int ellm_attn_merge_partials(const float* o_parts, const float* lse_parts, size_t parts,
                             size_t rows, size_t head_size, void* out, float* lse_out,
                             int device, void* stream);

/* Same combine with an fp32 result (out [rows, head_size] fp32): the local pre-merge of a
 * rank that holds several key chunks, before its partial travels to the rows' owner. */
int ellm_attn_merge_partials_f32(const float* o_parts, const float* lse_parts, size_t parts,
                                 size_t rows, size_t head_size, float* out, float* lse_out,
                                 int device, void* stream);

/* Attention over an explicit key window, fp32 partial output: chunk rows attend
 * keys [key_begin, min(key_end, position+1)) only.  Used by sequence-chunk
 * sharding, where each GPU holds one contiguous slice of the keys.
 * o_part [chunk rows, max_batch, q_heads, head_size] fp32, lse_part fp32. */
int ellm_attn_run_window(ellm_attn* h, size_t position_index, size_t position_interval,
                         size_t batch_size, size_t key_begin, size_t key_end, float* o_part,
                         float* lse_part);

/* ellm_attn_run_window with the queries read from `q` instead of the handle's bound q buffer
 * (same shape and strides; NULL = the bound buffer).  Sequence-chunk sharding gathers every
 * rank's query chunks into one buffer and runs each (query chunk, key chunk) pair straight from
 * it.  No counterpart in the reference (src/compiler/mul/attention.rs:41-67 binds q once). */
int ellm_attn_run_window_q(ellm_attn* h, const void* q, size_t position_index,
                           size_t position_interval, size_t batch_size, size_t key_begin,
                           size_t key_end, float* o_part, float* lse_part);

/* ellm_attn_merge_partials over parts that live in separate buffers: o_parts[i] [rows,
 * head_size] fp32 and lse_parts[i] [rows] fp32 are device pointers held in HOST arrays of
 * `parts` <= 16 entries; out is fp32 when out_is_f32 != 0, else bf16.  Lets partial results be
 * combined where they were computed or received, without gathering them first. */
int ellm_attn_merge_partials_list(const float* const* o_parts, const float* const* lse_parts,
                                  size_t parts, size_t rows, size_t head_size, void* out,
                                  int out_is_f32, float* lse_out, int device, void* stream);

/* For handles created with async = 1, whose run calls only enqueue: waits for the handle's
 * stream and returns ELLM_ERR_DEVICE_TIMEOUT if a bounded device-side wait of any kernel
 * launched since the last check ran out (the results of those calls are then invalid), else
 * ELLM_OK.  The counterpart of the executor's barrier after an operator
 * (src/serving/start.rs:69-73) for callers that synchronise once per step instead of once per
 * operator; same role as ellm_matmul_check for the projections. */
int ellm_attn_check(ellm_attn* h);

/* ---- Running a whole step without a host barrier per operator ----------------------------------
 * The reference's executor meets a barrier after every operator (src/serving/start.rs:69-73).
 * On a device the operators of a step can instead be enqueued back to back on one stream by
 * handles created with async = 1, with one wait per step - or, for decode steps, captured once
 * into a CUDA graph and replayed, every operator taking the sequences' positions from a device
 * array that the graph itself advances (ellm_attn_run_ragged / ellm_matmul3_run_ragged).  These
 * entry points give a host that has no CUDA binding of its own what it needs for that: a stream,
 * the wait, the position array's update, and the capture.  The stepping they serve is the one
 * the reference keeps in src/serving/start copy.rs:84-110.
 *
 * ellm_positions_set: positions[i] = value (add == 0) or positions[i] += value (add != 0) for
 * i < count, on the stream.  ellm_step_graph_begin .. ellm_step_graph_end bracket the run calls
 * of one step on `stream` (made by ellm_stream_create; every operator of the step must be an
 * async = 1 handle on that stream and must have run at least once before, outside a capture);
 * nothing executes in between, the calls are recorded.  ellm_step_graph_launch replays them. */
typedef struct ellm_step_graph ellm_step_graph;
int ellm_stream_create(int device, void** stream);
int ellm_stream_destroy(int device, void* stream);
int ellm_stream_synchronize(int device, void* stream);
int ellm_positions_set(int32_t* positions, size_t count, int32_t value, int add, int device,
                       void* stream);
int ellm_step_graph_begin(int device, void* stream);
int ellm_step_graph_end(int device, void* stream, ellm_step_graph** out);
int ellm_step_graph_launch(ellm_step_graph* graph, void* stream);
int ellm_step_graph_nodes(const ellm_step_graph* graph, size_t* nodes);   /* kernels recorded */
int ellm_step_graph_destroy(ellm_step_graph* graph);

/* Counters for the benchmark: kernels launched by this handle since creation, and
 * per-kernel device time when profiling is on (events around each launch). */
typedef enum ellm_kernel_id {
    ELLM_KERNEL_KV_APPEND = 0,
    ELLM_KERNEL_DECODE_SPLITKV = 1,
    ELLM_KERNEL_MERGE = 2,
    ELLM_KERNEL_PREFILL_TCGEN05 = 3,
    ELLM_KERNEL_PREFILL_WARP_MMA = 4,
    ELLM_KERNEL_COUNT = 5
} ellm_kernel_id;
int ellm_attn_set_profiling(ellm_attn* h, int on);
/* launches: all launches of that kernel; timed_launches / total_ms: those made while
 * profiling was on and their summed device time.  Synchronises the stream. */
int ellm_attn_kernel_stats(ellm_attn* h, int kernel_id, uint64_t* launches,
                           uint64_t* timed_launches, double* total_ms);

/* Decode step (one query row per sequence, split-KV + merge) that allocates nothing.
 *
 * It has no counterpart in the reference; it exists for callers that cannot obtain
 * device memory at run time.  eLLM plans every buffer while the graph is built and
 * gives all memory out there, and a serving process often shares its GPU with a
 * framework whose caching allocator already holds the whole HBM: in both cases
 * cudaMalloc inside the step loop either is forbidden or simply fails, so
 * ellm_attn_create (which allocates a workspace per handle) is not an option.
 *
 * Instead of a handle's workspace this entry point keeps the split-KV partials in
 * one fixed array that is part of the library image (a file-scope __device__ array,
 * about 8.1 MB, held by every GPU that loads the library until the process exits).
 * The caller passes every input and output; no handle is involved and the call makes
 * no cudaMalloc / cudaFree and uses no allocating library routine.
 *
 * Limit: batch_size * kv_heads * ceil((q_heads / kv_heads) / 16) + 2 * (SMs of the
 * device) must not exceed ELLM_NOALLOC_MAX_SLOTS, and batch_size must not exceed
 * ELLM_NOALLOC_MAX_BATCH; larger requests return ELLM_ERR_UNSUPPORTED and touch
 * nothing.  (On a 148-SM B200: batch_size * kv_heads * head tiles <= 728.)
 *
 * The first call on a device looks the array's device address up and sets the
 * kernel's shared-memory attribute for that device; make that first call before any
 * stream capture begins.  That look-up (or any earlier call into this library on the
 * device) is also the moment the library's device image, array included, is loaded:
 * it is the one place where this entry point depends on free device memory, so make
 * the first call before another allocator takes the GPU's memory.  If none is left it
 * returns ELLM_ERR_NO_MEMORY.  All calls on one device share the array, and it keeps
 * whatever the previous call left in it.  Nothing in it has to start at zero - each
 * call writes every slot before reading it - so sequential calls on one stream are
 * independent of one another, but two calls whose kernels overlap on the GPU (two
 * streams, two host threads) race on the array: serialise them.
 *
 * Arguments as in ellm_attn_desc / ellm_attn_run_ragged: q, out [max-batch rows >=
 * batch_size, q_heads, head_size] bf16; lse [batch_size, q_heads] fp32 or NULL;
 * positions device int32[batch_size] or NULL (then position_index for all); sequence
 * b attends keys 0..=position_b, which must already be in the cache.  Enqueues on
 * `stream` and returns without waiting. */
#define ELLM_NOALLOC_MAX_SLOTS 1024
#define ELLM_NOALLOC_MAX_BATCH 1024
int ellm_attn_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                             float* lse, const int32_t* positions, size_t position_index,
                             size_t batch_size, size_t q_heads, size_t kv_heads, size_t head_size,
                             const size_t kv_strides[4], size_t max_seq, float scale, int device,
                             void* stream);

/* Named options of a handle.
 *   "tc_wait_timeout_ns"    bound of every device-side wait of the tcgen05 prefill kernel
 *                           (default 2 000 000 000); when one runs out the kernel sets a status
 *                           word, releases its resources and returns; the call that launched it
 *                           returns ELLM_ERR_DEVICE_TIMEOUT when the handle synchronises
 *                           (async = 0), and ellm_attn_check reports it for async = 1 handles.
 *   "tc_debug_skip_kv_item" test hook for that path: the kernel's loader never fetches ring item
 *                           N (0 = first K tile, 1 = first V tile, ...) so the wait on it runs
 *                           out; -1 (default) = off.  The context stays usable afterwards.
 *   "decode_early_stream"   1: a decode step's kernel builds its tile table and requests its first K/V
 *                           rows before it waits for the stream's previous kernel, so that its start
 *                           overlaps that kernel's end.  The caller vouches that the previous kernel in
 *                           the stream writes neither the positions nor cache rows below each sequence's
 *                           newest row, and (if it is not one of this library's) that it was itself
 *                           ordered after whatever does.  True for the decode steps of a layer stack -
 *                           the projection before attention writes only Q and the newest row - and for
 *                           back-to-back steps on resident inputs; default 0.  ellm_attn_run_host never
 *                           uses it (its staging kernel writes the positions).
 *   "tc_fuse_append"        prefill kernel: 1 (default) the chunk's K/V rows are read from k_new / v_new and
 *                           written into the cache by the attention kernel itself when the chunk starts on a
 *                           128-key boundary (one start for all sequences); 0 always runs the append kernel
 *                           first.  Same cache bits either way.
 *   "tc_persistent"         prefill kernel: -1 (default) / 1 one CTA per SM walking the work-item list,
 *                           0 one CTA per item; a tuning knob.
 *   "decode_ctas"           grid of the decode kernel, 1 .. 2 x SMs (default 2 x SMs, for which the
 *                           workspace is sized); a tuning knob.
 * Unknown names return ELLM_ERR_INVALID_ARG.  The reference has no counterpart (it aborts). */
int ellm_attn_set_option(ellm_attn* h, const char* name, long long value);

const char* ellm_last_error(void);   /* thread-local text of the last failure */
const char* ellm_status_string(int status);
int ellm_attn_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ELLM_ATTN_H */
