// C ABI of the attention path (see include/ellm_attn.h): argument checks, the
// handle, kernel selection and launches.  No torch types, no CPU fallback: every
// call either launches the CUDA kernels or returns an error status.
#include "../../include/ellm_attn.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <utility>
#include <vector>

#include "decode_splitkv.cuh"
#include "kv_append.cuh"
#include "merge_partials.cuh"
#include "prefill_warp_mma.cuh"
#include "prefill_tcgen05.cuh"
#include "qk_norm_rope_append.cuh"
#include "rms_norm.cuh"

namespace ellm {

// The inputs of a host-buffer decode step, fetched from page-locked host memory by one small kernel
// instead of one copy node per buffer: up to four (destination, source, bytes) ranges, bytes a
// multiple of 4, both ends 16-byte aligned.
struct StageIn {
    void* dst[4];
    const void* src[4];
    unsigned long long bytes[4];
    int n;
};

// The ranges form one flat list of 16-byte chunks; a thread requests all of its chunks (two per
// round, normally one in all: the launch sizes the grid to the list) and its tail words before it
// stores any of them, so a step pays one round trip over PCIe, not one per range.
__global__ void __launch_bounds__(256) stage_in_kernel(const StageIn s) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const unsigned long long tid = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const unsigned long long step = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
    unsigned long long first[5];
    first[0] = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) first[k + 1] = first[k] + (k < s.n ? s.bytes[k] / 16 : 0);
    auto locate = [&](unsigned long long f, const uint4*& src, uint4*& dst) {
        src = static_cast<const uint4*>(s.src[0]) + f;
        dst = static_cast<uint4*>(s.dst[0]) + f;
#pragma unroll
        for (int k = 1; k < 4; ++k)
            if (k < s.n && f >= first[k]) {
                src = static_cast<const uint4*>(s.src[k]) + (f - first[k]);
                dst = static_cast<uint4*>(s.dst[k]) + (f - first[k]);
            }
    };
    // tail words of ranges whose size is not a multiple of 16 bytes
    unsigned tail[4];
    bool has_tail[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        has_tail[k] = k < s.n && tid < (s.bytes[k] % 16) / 4;
        if (has_tail[k]) tail[k] = static_cast<const unsigned*>(s.src[k])[(s.bytes[k] / 16) * 4 + tid];
    }
    for (unsigned long long f = tid; f < first[4]; f += 2 * step) {
        const uint4 *src_a, *src_b;
        uint4 *dst_a, *dst_b;
        locate(f, src_a, dst_a);
        const bool two = f + step < first[4];
        if (two) locate(f + step, src_b, dst_b);
        const uint4 a = *src_a;
        uint4 b = make_uint4(0u, 0u, 0u, 0u);
        if (two) b = *src_b;
        *dst_a = a;
        if (two) *dst_b = b;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k)
        if (has_tail[k]) static_cast<unsigned*>(s.dst[k])[(s.bytes[k] / 16) * 4 + tid] = tail[k];
}

}  // namespace ellm

namespace {

thread_local char g_err[512] = "";

int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return status;
}

#define ELLM_CUDA(call)                                                                      \
    do {                                                                                     \
        cudaError_t e_ = (call);                                                             \
        if (e_ != cudaSuccess)                                                               \
            return fail(ELLM_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), \
                        __FILE__, __LINE__);                                                 \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    }
    ~DeviceGuard() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Launch as a programmatic dependent of the stream's previous kernel: the grid may be set up
// while that kernel still runs, and waits for it on the device (griddepcontrol.wait at the top of
// the kernel) before it touches memory.  Hides launch latency between the small kernels of a
// decode step.  Only for kernels that do that wait.
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace

struct ellm_attn {
    ellm_attn_desc d;
    cudaStream_t stream = nullptr;
    int sm_count = 0;
    int group = 1, gtiles = 1;
    int dec_ctas = 0;
    size_t slots = 0;
    float* part_o = nullptr;           // two copies of the split-KV workspace, used in turn: a step's merge may
    float* part_lse = nullptr;         // still read one while the next step's decode kernel fills the other
    unsigned part_turn = 0;
    int decode_early = 0;              // ellm_attn_set_option("decode_early_stream")
    int32_t* positions_dev = nullptr;  // staging for ellm_attn_run_host
    int* status_dev = nullptr;         // bounded-wait status word written by the tcgen05 kernel; two more words behind it
                                       // are the prefill kernel's work-list counters
    int* status_host = nullptr;        // pinned mirror
    ellm::Tcgen05Plan tc;              // tensor maps etc. of the tcgen05 prefill kernel
    std::mutex mu;
    uint64_t launches[ELLM_KERNEL_COUNT] = {};
    uint64_t timed[ELLM_KERNEL_COUNT] = {};
    double total_ms[ELLM_KERNEL_COUNT] = {};
    bool profiling = false;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pending[ELLM_KERNEL_COUNT];
    // ellm_attn_run_host, decode with per-sequence positions: the copies and kernels of a step are
    // captured once into a CUDA graph and replayed while the caller's buffers stay the same
    struct HostStepKey {
        const void *q = nullptr, *k = nullptr, *v = nullptr, *out = nullptr, *lse = nullptr, *pos = nullptr;
        size_t batch = 0;
        bool operator==(const HostStepKey& o) const {
            return q == o.q && k == o.k && v == o.v && out == o.out && lse == o.lse && pos == o.pos && batch == o.batch;
        }
    } graph_key;
    cudaGraphExec_t graph_exec = nullptr;
    cudaStream_t graph_stream = nullptr;    // own stream: the caller's may be the legacy default stream, which cannot be captured
    cudaEvent_t graph_event = nullptr;
    uint64_t graph_launches[ELLM_KERNEL_COUNT] = {};
    bool graph_disabled = false;
    bool graph_key_rejected = false;        // graph_key names buffers that are not page-locked
};

namespace {

struct LaunchScope {  // counts a launch and, when profiling, brackets it with events
    ellm_attn* h;
    int id;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    LaunchScope(ellm_attn* h_, int id_) : h(h_), id(id_) {
        if (h && h->profiling) {
            cudaEventCreate(&e0);
            cudaEventCreate(&e1);
            cudaEventRecord(e0, h->stream);
        }
    }
    ~LaunchScope() {
        if (!h) return;
        h->launches[id]++;
        if (e0) {
            cudaEventRecord(e1, h->stream);
            h->pending[id].emplace_back(e0, e1);
        }
    }
};

int check_desc(const ellm_attn_desc* d) {
    if (!d) return fail(ELLM_ERR_INVALID_ARG, "desc is NULL");
    if (!d->q || !d->k_cache || !d->v_cache || !d->out)
        return fail(ELLM_ERR_INVALID_ARG, "q, k_cache, v_cache and out must be non-NULL");
    if ((d->k_new == nullptr) != (d->v_new == nullptr))
        return fail(ELLM_ERR_INVALID_ARG, "k_new and v_new must be both set or both NULL");
    if (d->dtype != ELLM_DTYPE_BF16) return fail(ELLM_ERR_UNSUPPORTED, "dtype %d: only bf16", d->dtype);
    if (d->head_size != static_cast<size_t>(ellm::kHeadDim))
        return fail(ELLM_ERR_UNSUPPORTED, "head_size %zu: only 128 (as the reference's f16 kernel)", d->head_size);
    if (d->max_batch == 0 || d->q_heads == 0 || d->kv_heads == 0 || d->max_seq == 0 || d->max_interval == 0)
        return fail(ELLM_ERR_INVALID_ARG, "max_batch, q_heads, kv_heads, max_seq, max_interval must be > 0");
    if (d->q_heads % d->kv_heads != 0)
        return fail(ELLM_ERR_INVALID_ARG, "q_heads %zu is not a multiple of kv_heads %zu", d->q_heads, d->kv_heads);
    if (d->kv_strides[3] != 1) return fail(ELLM_ERR_UNSUPPORTED, "kv_strides[3] must be 1 (head_dim contiguous)");
    for (int i = 0; i < 3; ++i)
        if (d->kv_strides[i] % 8 != 0 || d->kv_strides[i] == 0)
            return fail(ELLM_ERR_INVALID_ARG, "kv_strides[%d] = %zu must be a non-zero multiple of 8 elements", i, d->kv_strides[i]);
    if (!aligned16(d->q) || !aligned16(d->k_cache) || !aligned16(d->v_cache) || !aligned16(d->out) ||
        !aligned16(d->k_new) || !aligned16(d->v_new))
        return fail(ELLM_ERR_INVALID_ARG, "device buffers must be 16-byte aligned");
    if (d->lse && (reinterpret_cast<uintptr_t>(d->lse) & 3u)) return fail(ELLM_ERR_INVALID_ARG, "lse misaligned");
    if (!(d->scale > 0.0f) || !std::isfinite(d->scale)) return fail(ELLM_ERR_INVALID_ARG, "scale must be finite and > 0");
    if (d->prefill_kernel < ELLM_PREFILL_AUTO || d->prefill_kernel > ELLM_PREFILL_WARP_MMA)
        return fail(ELLM_ERR_INVALID_ARG, "prefill_kernel %d unknown", d->prefill_kernel);
    return ELLM_OK;
}

int launch_append(ellm_attn* h, cudaStream_t stream, void* k_cache, void* v_cache, const void* k_new,
                  const void* v_new, const size_t* strides, size_t max_batch, size_t kv_heads,
                  size_t max_seq, size_t position_index, const int32_t* positions, size_t interval,
                  size_t batch) {
    ellm::AppendParams ap;
    ap.k_new = static_cast<const uint4*>(k_new);
    ap.v_new = static_cast<const uint4*>(v_new);
    ap.k_cache = static_cast<__nv_bfloat16*>(k_cache);
    ap.v_cache = static_cast<__nv_bfloat16*>(v_cache);
    ap.positions = positions;
    ap.position_index = static_cast<long long>(position_index);
    ap.s0 = strides[0]; ap.s1 = strides[1]; ap.s2 = strides[2];
    ap.max_seq = static_cast<long long>(max_seq);
    ap.interval = static_cast<int>(interval);
    ap.batch = static_cast<int>(batch);
    ap.max_batch = static_cast<int>(max_batch);
    ap.kv_heads = static_cast<int>(kv_heads);
    const long long threads = static_cast<long long>(interval) * batch * kv_heads * 16;
    const unsigned blocks = static_cast<unsigned>((threads + 255) / 256);
    {
        LaunchScope ls(h, ELLM_KERNEL_KV_APPEND);
        ellm::kv_append_kernel<<<blocks, 256, 0, stream>>>(ap);
    }
    ELLM_CUDA(cudaGetLastError());
    return ELLM_OK;
}

// The merge of a decode step in the shape that fits the step: many rows with few pieces each get
// the light shape (2 warps per row, tables in dynamic shared memory), few rows with many pieces the
// wide one.  A row's pieces are at most the decode grid's CTAs.
cudaError_t launch_merge(const ellm::DecodeParams& p, size_t batch, unsigned blocks, float* out_f32, void* out_bf16,
                         float* lse_out, cudaStream_t stream, bool dependent) {
    const int pieces_cap = std::min(p.num_ctas, ellm::kMergeMaxPieces);
    const size_t smem = ellm::merge_smem_bytes(static_cast<int>(batch), pieces_cap);
    const bool light = blocks >= 128;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(light ? ellm::kMergeLightThreads : ellm::kMergeThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent ? 1 : 0;
    __nv_bfloat16* ob = static_cast<__nv_bfloat16*>(out_bf16);
    if (out_f32)
        return light ? cudaLaunchKernelEx(&cfg, ellm::decode_merge_kernel<float, 2, 4>, p, out_f32, lse_out, pieces_cap)
                     : cudaLaunchKernelEx(&cfg, ellm::decode_merge_kernel<float, 8, 10>, p, out_f32, lse_out, pieces_cap);
    return light ? cudaLaunchKernelEx(&cfg, ellm::decode_merge_kernel<__nv_bfloat16, 2, 4>, p, ob, lse_out, pieces_cap)
                 : cudaLaunchKernelEx(&cfg, ellm::decode_merge_kernel<__nv_bfloat16, 8, 10>, p, ob, lse_out, pieces_cap);
}

// Decode (interval == 1): K2 then K3.  out_f32 != nullptr selects the fp32
// partial output of the windowed form.
int launch_decode(ellm_attn* h, const int32_t* positions, size_t position_index, size_t batch,
                  long long key_begin, long long key_end, float* out_f32, float* lse_out, bool append,
                  void* out_override = nullptr, bool early = false) {
    if (batch > static_cast<size_t>(ellm::kDecMaxBatch))
        return fail(ELLM_ERR_UNSUPPORTED, "decode batch %zu exceeds %d", batch, ellm::kDecMaxBatch);
    ellm::DecodeParams p;
    p.q = static_cast<const __nv_bfloat16*>(h->d.q);
    p.k_cache = static_cast<const __nv_bfloat16*>(h->d.k_cache);
    p.v_cache = static_cast<const __nv_bfloat16*>(h->d.v_cache);
    h->part_turn ^= 1u;
    p.part_o = h->part_o + (h->part_turn ? h->slots * 16 * ellm::kHeadDim : 0);
    p.part_lse = h->part_lse + (h->part_turn ? h->slots * 16 : 0);
    p.early = early ? 1 : 0;
    p.positions = positions;
    long long len = static_cast<long long>(position_index) + 1;
    if (len > key_end) len = key_end;
    p.uniform_len = len;
    p.len_cap = key_end < static_cast<long long>(h->d.max_seq) ? key_end : static_cast<long long>(h->d.max_seq);
    p.key_begin = key_begin;
    p.s0 = h->d.kv_strides[0]; p.s1 = h->d.kv_strides[1]; p.s2 = h->d.kv_strides[2];
    p.batch = static_cast<int>(batch);
    p.q_heads = static_cast<int>(h->d.q_heads);
    p.kv_heads = static_cast<int>(h->d.kv_heads);
    p.group = h->group;
    p.gtiles = h->gtiles;
    p.scale_log2 = h->d.scale * ellm::kLog2e;
    p.num_ctas = h->dec_ctas;
    if (append) {   // the new token's K/V rows ride along with the decode kernel
        p.k_new = static_cast<const __nv_bfloat16*>(h->d.k_new);
        p.v_new = static_cast<const __nv_bfloat16*>(h->d.v_new);
        p.k_cache_w = static_cast<__nv_bfloat16*>(h->d.k_cache);
        p.v_cache_w = static_cast<__nv_bfloat16*>(h->d.v_cache);
    }
    {
        LaunchScope ls(h, ELLM_KERNEL_DECODE_SPLITKV);
        if (h->group <= 8)   // blocks of 8 query heads per segment: one for groups of up to 8 heads, else two
            launch_dependent(ellm::decode_splitkv_kernel<1>, h->dec_ctas, ellm::kDecThreads, ellm::kDecSmemBytes, h->stream, p);
        else
            launch_dependent(ellm::decode_splitkv_kernel<2>, h->dec_ctas, ellm::kDecThreads, ellm::kDecSmemBytes, h->stream, p);
    }
    ELLM_CUDA(cudaGetLastError());
    const unsigned blocks = static_cast<unsigned>(batch * h->d.q_heads);
    {
        // programmatic dependent launch: the merge grid is set up while the decode grid drains;
        // its first instruction waits for the decode grid's memory to be visible
        LaunchScope ls(h, ELLM_KERNEL_MERGE);
        const cudaError_t e = launch_merge(p, batch, blocks, out_f32, out_f32 ? nullptr : (out_override ? out_override : h->d.out),
                                           lse_out, h->stream, true);
        if (e != cudaSuccess) return fail(ELLM_ERR_CUDA, "merge launch failed: %s", cudaGetErrorString(e));
    }
    ELLM_CUDA(cudaGetLastError());
    return ELLM_OK;
}

int launch_prefill_warp_mma(ellm_attn* h, const int32_t* positions, size_t position_index,
                            size_t interval, size_t batch, long long key_begin, long long key_end,
                            float* out_f32, float* lse_out) {
    ellm::PrefillParams p;
    p.q = static_cast<const __nv_bfloat16*>(h->d.q);
    p.k_cache = static_cast<const __nv_bfloat16*>(h->d.k_cache);
    p.v_cache = static_cast<const __nv_bfloat16*>(h->d.v_cache);
    p.out = out_f32 ? static_cast<void*>(out_f32) : h->d.out;
    p.lse = lse_out;
    p.positions = positions;
    p.position_index = static_cast<long long>(position_index);
    p.key_begin = key_begin;
    p.key_end = key_end < static_cast<long long>(h->d.max_seq) ? key_end : static_cast<long long>(h->d.max_seq);
    p.s0 = h->d.kv_strides[0]; p.s1 = h->d.kv_strides[1]; p.s2 = h->d.kv_strides[2];
    p.interval = static_cast<int>(interval);
    p.batch = static_cast<int>(batch);
    p.max_batch = static_cast<int>(h->d.max_batch);
    p.q_heads = static_cast<int>(h->d.q_heads);
    p.kv_heads = static_cast<int>(h->d.kv_heads);
    p.group = h->group;
    p.row_tiles = static_cast<int>((interval * h->group + ellm::kPfRows - 1) / ellm::kPfRows);
    p.scale_log2 = h->d.scale * ellm::kLog2e;
    if (batch > 65535 || h->d.kv_heads > 65535)
        return fail(ELLM_ERR_UNSUPPORTED, "batch / kv_heads exceed the grid limit 65535");
    dim3 grid(p.row_tiles, p.kv_heads, p.batch);
    {
        LaunchScope ls(h, ELLM_KERNEL_PREFILL_WARP_MMA);
        if (out_f32)
            ellm::prefill_warp_mma_kernel<float><<<grid, ellm::kPfThreads, ellm::kPfSmemBytes, h->stream>>>(p);
        else
            ellm::prefill_warp_mma_kernel<__nv_bfloat16><<<grid, ellm::kPfThreads, ellm::kPfSmemBytes, h->stream>>>(p);
    }
    ELLM_CUDA(cudaGetLastError());
    return ELLM_OK;
}

// [rows][pitch bytes] block of which `width` bytes per row are live: one flat copy when the rows are
// contiguous (live batch == allocated batch), a pitched copy otherwise.
cudaError_t copy_rows(void* dst, const void* src, size_t pitch, size_t width, size_t rows, cudaMemcpyKind kind,
                      cudaStream_t stream) {
    if (width == pitch || rows == 1) return cudaMemcpyAsync(dst, src, rows == 1 ? width : pitch * rows, kind, stream);
    return cudaMemcpy2DAsync(dst, pitch, src, pitch, width, rows, kind, stream);
}

int finish(ellm_attn* h, bool enqueue_only) {
    if (enqueue_only) return ELLM_OK;
    ELLM_CUDA(cudaStreamSynchronize(h->stream));
    if (h->status_host && *h->status_host != 0) {
        const int code = *h->status_host;
        *h->status_host = 0;
        cudaMemsetAsync(h->status_dev, 0, 4 * sizeof(int), h->stream);   // the status word and the work-list counters
        return fail(ELLM_ERR_DEVICE_TIMEOUT, "a bounded device-side wait ran out (code %d)", code);
    }
    return ELLM_OK;
}

// Common body of run / run_ragged / run_window.
int run_impl(ellm_attn* h, const int32_t* positions, size_t position_index, size_t interval,
             size_t batch, long long key_begin, long long key_end, float* out_f32, float* lse_out,
             bool append, int enqueue_only = -1, const cudaStream_t* stream_override = nullptr,
             void* decode_out_override = nullptr, const void* q_override = nullptr) {
    if (!h) return fail(ELLM_ERR_INVALID_ARG, "handle is NULL");
    if (interval == 0 || batch == 0) return ELLM_OK;  // nothing to do, as an empty assign() range
    if (batch > h->d.max_batch) return fail(ELLM_ERR_INVALID_ARG, "batch_size %zu > max_batch %zu", batch, h->d.max_batch);
    if (interval > h->d.max_interval)
        return fail(ELLM_ERR_INVALID_ARG, "position_interval %zu > max_interval %zu", interval, h->d.max_interval);
    if (key_begin < 0 || key_end < key_begin) return fail(ELLM_ERR_INVALID_ARG, "bad key window");
    // a windowed call may place its rows past the cache (a later chunk of a sharded sequence
    // attending an earlier chunk's keys): only the keys it reads must be inside the cache
    if (!positions && position_index + interval > h->d.max_seq && key_end > static_cast<long long>(h->d.max_seq))
        return fail(ELLM_ERR_INVALID_ARG, "position_index %zu + interval %zu exceeds max_seq %zu", position_index, interval, h->d.max_seq);
    DeviceGuard guard(h->d.device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", h->d.device);
    std::lock_guard<std::mutex> lock(h->mu);
    // a caller may direct this one step to another stream (the host-buffer entry point's graph
    // stream); the handle's stream is put back before the lock is released
    struct StreamSwap {
        ellm_attn* h;
        cudaStream_t saved;
        StreamSwap(ellm_attn* h_, const cudaStream_t* o) : h(h_), saved(h_->stream) { if (o) h->stream = *o; }
        ~StreamSwap() { h->stream = saved; }
    } swap(h, stream_override);
    // a windowed call may read its queries from another buffer of the same shape (the gathered
    // query chunks of a sharded sequence): the handle's q is put back before the lock is released
    struct QuerySwap {
        ellm_attn* h;
        const void* saved;
        QuerySwap(ellm_attn* h_, const void* q) : h(h_), saved(h_->d.q) { if (q) h->d.q = q; }
        ~QuerySwap() { h->d.q = saved; }
    } qswap(h, q_override);
    const bool no_sync = enqueue_only < 0 ? h->d.async != 0 : enqueue_only != 0;
    int rc;
    const bool do_append = append && h->d.k_new;
    // which kernel takes a chunk of more than one row
    bool use_tc = false;
    if (interval > 1) {
        if (h->d.prefill_kernel == ELLM_PREFILL_TCGEN05) use_tc = true;
        else if (h->d.prefill_kernel == ELLM_PREFILL_AUTO) use_tc = ellm::tcgen05_prefers(h->tc, interval, h->group);
    }
    // the chunk's K/V rows go into the cache inside the attention kernel where that is possible (a decode
    // step always does; the tensor-memory prefill kernel when the chunk starts on a key-tile boundary),
    // else by the append kernel first
    const bool fused = use_tc && do_append && !out_f32 &&
                       ellm::tcgen05_can_fuse_append(h->tc, h->d, positions, position_index, batch, key_begin, key_end);
    if (do_append && interval > 1 && !fused) {
        rc = launch_append(h, h->stream, h->d.k_cache, h->d.v_cache, h->d.k_new, h->d.v_new, h->d.kv_strides,
                           h->d.max_batch, h->d.kv_heads, h->d.max_seq, position_index, positions, interval, batch);
        if (rc) return rc;
    }
    if (interval == 1) {
        // early streaming only where the caller vouched for it, and never for a step whose inputs the
        // library itself stages right before (the host-buffer entry point passes a stream override)
        rc = launch_decode(h, positions, position_index, batch, key_begin, key_end, out_f32, lse_out, do_append,
                           decode_out_override, h->decode_early != 0 && stream_override == nullptr);
    } else {
        if (use_tc) {
            if (!h->tc.ready)
                return fail(ELLM_ERR_UNSUPPORTED, "tcgen05 prefill unavailable for this handle: %s", h->tc.why);
            {
                LaunchScope ls(h, ELLM_KERNEL_PREFILL_TCGEN05);
                rc = ellm::launch_prefill_tcgen05(h->tc, h->d, positions, position_index, interval, batch, key_begin, key_end,
                                                  out_f32, lse_out, h->status_dev, h->stream, fused);
            }
            if (rc == ELLM_ERR_UNSUPPORTED) return fail(rc, "tcgen05 prefill: %s", h->tc.why);
            if (rc) return fail(rc, "tcgen05 prefill launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        } else {
            rc = launch_prefill_warp_mma(h, positions, position_index, interval, batch, key_begin, key_end, out_f32, lse_out);
        }
    }
    if (rc) return rc;
    if (h->status_dev && !no_sync && interval > 1)
        cudaMemcpyAsync(h->status_host, h->status_dev, sizeof(int), cudaMemcpyDeviceToHost, h->stream);
    return finish(h, no_sync);
}

}  // namespace

extern "C" {

int ellm_attn_abi_version(void) { return 1; }

const char* ellm_last_error(void) { return g_err; }

const char* ellm_status_string(int status) {
    switch (status) {
        case ELLM_OK: return "ok";
        case ELLM_ERR_INVALID_ARG: return "invalid argument";
        case ELLM_ERR_CUDA: return "CUDA error";
        case ELLM_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
        case ELLM_ERR_UNSUPPORTED: return "unsupported shape";
        case ELLM_ERR_NO_MEMORY: return "out of memory";
        default: return "unknown status";
    }
}

int ellm_attn_create(const ellm_attn_desc* desc, ellm_attn** out) {
    if (!out) return fail(ELLM_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    int rc = check_desc(desc);
    if (rc) return rc;
    int ndev = 0;
    ELLM_CUDA(cudaGetDeviceCount(&ndev));
    if (desc->device < 0 || desc->device >= ndev)
        return fail(ELLM_ERR_INVALID_ARG, "device %d out of range (%d devices)", desc->device, ndev);
    DeviceGuard guard(desc->device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", desc->device);
    cudaDeviceProp prop;
    ELLM_CUDA(cudaGetDeviceProperties(&prop, desc->device));
    if (prop.major != 10)
        return fail(ELLM_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", desc->device, prop.major, prop.minor);
    ellm_attn* h = new (std::nothrow) ellm_attn();
    if (!h) return fail(ELLM_ERR_NO_MEMORY, "host allocation failed");
    h->d = *desc;
    h->stream = static_cast<cudaStream_t>(desc->stream);
    h->sm_count = prop.multiProcessorCount;
    h->group = static_cast<int>(desc->q_heads / desc->kv_heads);
    h->gtiles = (h->group + 15) / 16;
    h->dec_ctas = 2 * h->sm_count;
    h->slots = static_cast<size_t>(h->dec_ctas) + desc->max_batch * desc->kv_heads * h->gtiles;
    auto cleanup = [&](int status) {
        ellm_attn_destroy(h);
        return status;
    };
    if (cudaMalloc(&h->part_o, 2 * h->slots * 16 * ellm::kHeadDim * sizeof(float)) != cudaSuccess ||
        cudaMalloc(&h->part_lse, 2 * h->slots * 16 * sizeof(float)) != cudaSuccess ||
        cudaMalloc(&h->positions_dev, desc->max_batch * sizeof(int32_t)) != cudaSuccess ||
        cudaMalloc(&h->status_dev, 4 * sizeof(int)) != cudaSuccess ||
        cudaMallocHost(&h->status_host, sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return cleanup(fail(ELLM_ERR_NO_MEMORY, "workspace allocation failed (%zu slots)", h->slots));
    }
    *h->status_host = 0;
    if (cudaMemset(h->status_dev, 0, 4 * sizeof(int)) != cudaSuccess) return cleanup(fail(ELLM_ERR_CUDA, "memset failed"));
    if (cudaFuncSetAttribute(ellm::decode_splitkv_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, ellm::kDecSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(ellm::decode_splitkv_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, ellm::kDecSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(ellm::prefill_warp_mma_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, ellm::kPfSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(ellm::prefill_warp_mma_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, ellm::kPfSmemBytes) != cudaSuccess)
        return cleanup(fail(ELLM_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(cudaGetLastError())));
    h->tc.sched = h->status_dev + 2;
    ellm::tcgen05_plan_init(h->tc, h->d, h->sm_count);  // leaves tc.ready false (with a reason) when it cannot serve this handle
    if (desc->prefill_kernel == ELLM_PREFILL_TCGEN05 && !h->tc.ready) {
        fail(ELLM_ERR_UNSUPPORTED, "tcgen05 prefill requested but unavailable: %s", h->tc.why);
        return cleanup(ELLM_ERR_UNSUPPORTED);
    }
    *out = h;
    return ELLM_OK;
}

int ellm_attn_destroy(ellm_attn* h) {
    if (!h) return ELLM_OK;
    DeviceGuard guard(h->d.device);
    for (auto& v : h->pending)
        for (auto& pr : v) {
            cudaEventDestroy(pr.first);
            cudaEventDestroy(pr.second);
        }
    if (h->graph_exec) cudaGraphExecDestroy(h->graph_exec);
    if (h->graph_event) cudaEventDestroy(h->graph_event);
    if (h->graph_stream) cudaStreamDestroy(h->graph_stream);
    cudaFree(h->part_o);
    cudaFree(h->part_lse);
    cudaFree(h->positions_dev);
    cudaFree(h->status_dev);
    if (h->status_host) cudaFreeHost(h->status_host);
    delete h;
    return ELLM_OK;
}

int ellm_attn_run(ellm_attn* h, size_t position_index, size_t position_interval, size_t batch_size,
                  size_t cpu_num, size_t thread_id) {
    if (!h) return fail(ELLM_ERR_INVALID_ARG, "handle is NULL");
    if (cpu_num == 0 || thread_id >= cpu_num) return fail(ELLM_ERR_INVALID_ARG, "thread_id %zu outside cpu_num %zu", thread_id, cpu_num);
    if (thread_id != 0) return ELLM_OK;  // one launch per operator step; the others go straight to the barrier
    return run_impl(h, nullptr, position_index, position_interval, batch_size, 0, INT64_MAX, nullptr, h->d.lse, true);
}

int ellm_attn_run_ragged(ellm_attn* h, const int32_t* positions, size_t position_interval,
                         size_t batch_size, size_t cpu_num, size_t thread_id) {
    if (!h) return fail(ELLM_ERR_INVALID_ARG, "handle is NULL");
    if (!positions) return fail(ELLM_ERR_INVALID_ARG, "positions is NULL");
    if (cpu_num == 0 || thread_id >= cpu_num) return fail(ELLM_ERR_INVALID_ARG, "thread_id %zu outside cpu_num %zu", thread_id, cpu_num);
    if (thread_id != 0) return ELLM_OK;
    return run_impl(h, positions, 0, position_interval, batch_size, 0, INT64_MAX, nullptr, h->d.lse, true);
}

int ellm_attn_run_window(ellm_attn* h, size_t position_index, size_t position_interval,
                         size_t batch_size, size_t key_begin, size_t key_end, float* o_part,
                         float* lse_part) {
    if (!o_part || !lse_part) return fail(ELLM_ERR_INVALID_ARG, "o_part and lse_part must be non-NULL");
    return run_impl(h, nullptr, position_index, position_interval, batch_size, static_cast<long long>(key_begin),
                    static_cast<long long>(key_end > static_cast<size_t>(INT64_MAX) ? INT64_MAX : key_end), o_part, lse_part, false);
}

int ellm_attn_run_window_q(ellm_attn* h, const void* q, size_t position_index, size_t position_interval,
                           size_t batch_size, size_t key_begin, size_t key_end, float* o_part, float* lse_part) {
    if (!o_part || !lse_part) return fail(ELLM_ERR_INVALID_ARG, "o_part and lse_part must be non-NULL");
    if (q && !aligned16(q)) return fail(ELLM_ERR_INVALID_ARG, "q must be 16-byte aligned");
    return run_impl(h, nullptr, position_index, position_interval, batch_size, static_cast<long long>(key_begin),
                    static_cast<long long>(key_end > static_cast<size_t>(INT64_MAX) ? INT64_MAX : key_end), o_part, lse_part, false,
                    -1, nullptr, nullptr, q);
}

int ellm_attn_check(ellm_attn* h) {
    if (!h) return fail(ELLM_ERR_INVALID_ARG, "handle is NULL");
    DeviceGuard guard(h->d.device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", h->d.device);
    std::lock_guard<std::mutex> lock(h->mu);
    if (h->status_dev)
        ELLM_CUDA(cudaMemcpyAsync(h->status_host, h->status_dev, sizeof(int), cudaMemcpyDeviceToHost, h->stream));
    return finish(h, false);
}

int ellm_attn_run_host(ellm_attn* h, const void* q_host, const void* k_new_host, const void* v_new_host,
                       void* out_host, float* lse_host, const int32_t* positions_host,
                       size_t position_index, size_t position_interval, size_t batch_size) {
    if (!h) return fail(ELLM_ERR_INVALID_ARG, "handle is NULL");
    if (!q_host || !out_host) return fail(ELLM_ERR_INVALID_ARG, "q_host and out_host must be non-NULL");
    if ((k_new_host || v_new_host) && !h->d.k_new) return fail(ELLM_ERR_INVALID_ARG, "handle has no k_new/v_new device buffers bound");
    if ((k_new_host == nullptr) != (v_new_host == nullptr)) return fail(ELLM_ERR_INVALID_ARG, "k_new_host and v_new_host must come together");
    if (lse_host && !h->d.lse) return fail(ELLM_ERR_INVALID_ARG, "handle has no lse device buffer bound");
    if (batch_size == 0 || position_interval == 0) return ELLM_OK;
    if (batch_size > h->d.max_batch || position_interval > h->d.max_interval)
        return fail(ELLM_ERR_INVALID_ARG, "batch_size / position_interval exceed the handle's maxima");
    DeviceGuard guard(h->d.device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", h->d.device);
    const size_t D = h->d.head_size;
    // [interval][max_batch][heads][D]: copy the live batch of every chunk row
    const size_t q_pitch = h->d.max_batch * h->d.q_heads * D * 2, q_width = batch_size * h->d.q_heads * D * 2;
    const size_t kv_pitch = h->d.max_batch * h->d.kv_heads * D * 2, kv_width = batch_size * h->d.kv_heads * D * 2;
    const size_t l_pitch = h->d.max_batch * h->d.q_heads * 4, l_width = batch_size * h->d.q_heads * 4;
    const uint64_t tc_before = h->launches[ELLM_KERNEL_PREFILL_TCGEN05];
    // The captured decode step moves its data without copy nodes: one small kernel fetches all
    // inputs from the page-locked host buffers, and the merge kernel writes O and LSE straight
    // into the host buffers (ordinary stores through the buffers' device addresses).
    auto enqueue_direct = [&](cudaStream_t stream) -> int {
        auto dev_ptr = [](const void* host, void** out) {
            *out = nullptr;
            if (!host) return true;
            if (reinterpret_cast<uintptr_t>(host) & 15u) return false;
            if (cudaHostGetDevicePointer(out, const_cast<void*>(host), 0) != cudaSuccess) { cudaGetLastError(); return false; }
            return (reinterpret_cast<uintptr_t>(*out) & 15u) == 0;
        };
        void *dq, *dk, *dv, *dp, *dout, *dlse;
        if (!dev_ptr(q_host, &dq) || !dev_ptr(k_new_host, &dk) || !dev_ptr(v_new_host, &dv) || !dev_ptr(positions_host, &dp) ||
            !dev_ptr(out_host, &dout) || !dev_ptr(lse_host, &dlse))
            return ELLM_ERR_UNSUPPORTED;
        ellm::StageIn si{};
        auto add = [&](const void* dst, const void* src, size_t bytes) {
            si.dst[si.n] = const_cast<void*>(dst); si.src[si.n] = src; si.bytes[si.n] = bytes; ++si.n;
        };
        add(h->d.q, dq, q_width);
        if (k_new_host) { add(h->d.k_new, dk, kv_width); add(h->d.v_new, dv, kv_width); }
        // (the positions are staged like the rest: letting the decode and merge kernels read them straight
        // from the page-locked buffer, to start streaming K/V while Q is still on its way, was measured -
        // every CTA's read is its own PCIe transaction, and 800 CTAs of them made the step 27 us longer)
        add(h->positions_dev, dp, batch_size * sizeof(int32_t));
        unsigned long long stage_chunks = 0;
        for (int i = 0; i < si.n; ++i) stage_chunks += si.bytes[i] / 16;
        const unsigned stage_blocks = static_cast<unsigned>(std::min<unsigned long long>(std::max<unsigned long long>((stage_chunks + 255) / 256, 1), 1184));
        ellm::stage_in_kernel<<<stage_blocks, 256, 0, stream>>>(si);
        ELLM_CUDA(cudaGetLastError());
        return run_impl(h, h->positions_dev, position_index, 1, batch_size, 0, INT64_MAX, nullptr,
                        lse_host ? static_cast<float*>(dlse) : h->d.lse, k_new_host != nullptr, /*enqueue_only=*/1, &stream, dout);
    };
    // everything a step enqueues on `stream`: inputs in, kernels, results out
    auto enqueue = [&](cudaStream_t stream) -> int {
        ELLM_CUDA(copy_rows(const_cast<void*>(h->d.q), q_host, q_pitch, q_width, position_interval, cudaMemcpyHostToDevice, stream));
        if (k_new_host) {
            ELLM_CUDA(copy_rows(const_cast<void*>(h->d.k_new), k_new_host, kv_pitch, kv_width, position_interval, cudaMemcpyHostToDevice, stream));
            ELLM_CUDA(copy_rows(const_cast<void*>(h->d.v_new), v_new_host, kv_pitch, kv_width, position_interval, cudaMemcpyHostToDevice, stream));
        }
        const int32_t* positions = nullptr;
        if (positions_host) {
            ELLM_CUDA(cudaMemcpyAsync(h->positions_dev, positions_host, batch_size * sizeof(int32_t), cudaMemcpyHostToDevice, stream));
            positions = h->positions_dev;
        }
        int rc = run_impl(h, positions, position_index, position_interval, batch_size, 0, INT64_MAX, nullptr, h->d.lse,
                          k_new_host != nullptr, /*enqueue_only=*/1, &stream);
        if (rc) return rc;
        ELLM_CUDA(copy_rows(out_host, h->d.out, q_pitch, q_width, position_interval, cudaMemcpyDeviceToHost, stream));
        if (lse_host)
            ELLM_CUDA(copy_rows(lse_host, h->d.lse, l_pitch, l_width, position_interval, cudaMemcpyDeviceToHost, stream));
        return ELLM_OK;
    };

    // Decode steps with per-sequence positions and pinned buffers repeat identically (only the
    // buffers' contents change), so the whole step is captured once and replayed.
    auto pinned = [](const void* ptr) {
        if (!ptr) return true;
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, ptr) != cudaSuccess) { cudaGetLastError(); return false; }
        return at.type == cudaMemoryTypeHost;
    };
    ellm_attn::HostStepKey key;
    key.q = q_host; key.k = k_new_host; key.v = v_new_host; key.out = out_host; key.lse = lse_host; key.pos = positions_host;
    key.batch = batch_size;
    bool use_graph = position_interval == 1 && positions_host && !h->profiling && !h->graph_disabled;
    if (use_graph && h->graph_key_rejected && h->graph_key == key) use_graph = false;
    if (use_graph && !(h->graph_exec && h->graph_key == key)) {
        // (re)build: the buffers must be page-locked for the copies to be captured
        if (h->graph_exec) { cudaGraphExecDestroy(h->graph_exec); h->graph_exec = nullptr; }
        use_graph = pinned(q_host) && pinned(k_new_host) && pinned(v_new_host) && pinned(out_host) && pinned(lse_host) &&
                    pinned(positions_host);
        h->graph_key = key;
        h->graph_key_rejected = !use_graph;
        if (use_graph && !h->graph_stream) {
            if (cudaStreamCreateWithFlags(&h->graph_stream, cudaStreamNonBlocking) != cudaSuccess ||
                cudaEventCreateWithFlags(&h->graph_event, cudaEventDisableTiming) != cudaSuccess) {
                cudaGetLastError();
                h->graph_disabled = true;
                use_graph = false;
            }
        }
        if (use_graph) {
            uint64_t before[ELLM_KERNEL_COUNT];
            for (int i = 0; i < ELLM_KERNEL_COUNT; ++i) before[i] = h->launches[i];
            cudaGraph_t graph = nullptr;
            bool ok = cudaStreamBeginCapture(h->graph_stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
            if (ok) {
                int rc = enqueue_direct(h->graph_stream);   // nothing is enqueued when it declines
                if (rc == ELLM_ERR_UNSUPPORTED) rc = enqueue(h->graph_stream);
                const cudaError_t e = cudaStreamEndCapture(h->graph_stream, &graph);
                ok = rc == ELLM_OK && e == cudaSuccess && graph != nullptr;
            }
            if (ok) ok = cudaGraphInstantiate(&h->graph_exec, graph, 0) == cudaSuccess;
            if (graph) cudaGraphDestroy(graph);
            for (int i = 0; i < ELLM_KERNEL_COUNT; ++i) {   // the capture launched nothing yet
                h->graph_launches[i] = h->launches[i] - before[i];
                h->launches[i] = before[i];
            }
            if (!ok) {
                cudaGetLastError();
                h->graph_exec = nullptr;
                h->graph_disabled = true;   // fall back to plain enqueues for this handle
                use_graph = false;
            } else {
                h->graph_key = key;
            }
        }
    }
    if (use_graph) {
        // replay in the caller's stream; the legacy default stream cannot take a graph launch that
        // must stay ordered with other streams' work, so there the graph runs in the handle's own
        // stream, ordered after whatever the caller queued
        const bool own = h->stream == nullptr || h->stream == cudaStreamLegacy || h->stream == cudaStreamPerThread;
        cudaStream_t run_stream = own ? h->graph_stream : h->stream;
        if (own) {
            ELLM_CUDA(cudaEventRecord(h->graph_event, h->stream));
            ELLM_CUDA(cudaStreamWaitEvent(h->graph_stream, h->graph_event, 0));
        }
        ELLM_CUDA(cudaGraphLaunch(h->graph_exec, run_stream));
        for (int i = 0; i < ELLM_KERNEL_COUNT; ++i) h->launches[i] += h->graph_launches[i];
        ELLM_CUDA(cudaStreamSynchronize(run_stream));
        return ELLM_OK;
    }

    int rc = enqueue(h->stream);
    if (rc) return rc;
    // only the tcgen05 kernel has device-side waits that can run out
    const bool read_status = h->launches[ELLM_KERNEL_PREFILL_TCGEN05] != tc_before;
    if (read_status) ELLM_CUDA(cudaMemcpyAsync(h->status_host, h->status_dev, sizeof(int), cudaMemcpyDeviceToHost, h->stream));
    ELLM_CUDA(cudaStreamSynchronize(h->stream));
    if (*h->status_host != 0) {
        const int code = *h->status_host;
        *h->status_host = 0;
        cudaMemsetAsync(h->status_dev, 0, 4 * sizeof(int), h->stream);
        return fail(ELLM_ERR_DEVICE_TIMEOUT, "a bounded device-side wait ran out (code %d)", code);
    }
    return ELLM_OK;
}

int ellm_device_alloc(int device, size_t bytes, void** out) {
    if (!out) return fail(ELLM_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    if (bytes == 0) return fail(ELLM_ERR_INVALID_ARG, "bytes is 0");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", device);
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {  // cudaMalloc returns at least 256-byte alignment
        cudaGetLastError();
        return fail(ELLM_ERR_NO_MEMORY, "cudaMalloc of %zu bytes failed", bytes);
    }
    if (cudaMemset(p, 0, bytes) != cudaSuccess) {
        cudaFree(p);
        return fail(ELLM_ERR_CUDA, "cudaMemset failed");
    }
    *out = p;
    return ELLM_OK;
}

int ellm_device_free(int device, void* ptr) {
    if (!ptr) return ELLM_OK;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", device);
    ELLM_CUDA(cudaFree(ptr));
    return ELLM_OK;
}

// The static KV cache as an object of the library: one zero-filled allocation for K and one for V,
// [layer, sequence, kv_head, position, head_size], never resized.
struct ellm_kv_cache {
    int device = 0;
    size_t layers = 0, max_batch = 0, kv_heads = 0, max_seq = 0, head_size = 0;
    size_t layer_elems = 0;
    void* k = nullptr;
    void* v = nullptr;
};

int ellm_kv_cache_create(int device, size_t layers, size_t max_batch, size_t kv_heads, size_t max_seq,
                         size_t head_size, ellm_kv_cache** out) {
    if (!out) return fail(ELLM_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    if (layers == 0 || max_batch == 0 || kv_heads == 0 || max_seq == 0)
        return fail(ELLM_ERR_INVALID_ARG, "layers, max_batch, kv_heads and max_seq must be > 0");
    if (head_size != static_cast<size_t>(ellm::kHeadDim)) return fail(ELLM_ERR_UNSUPPORTED, "head_size %zu: only 128", head_size);
    ellm_kv_cache* c = new (std::nothrow) ellm_kv_cache();
    if (!c) return fail(ELLM_ERR_NO_MEMORY, "host allocation failed");
    c->device = device;
    c->layers = layers; c->max_batch = max_batch; c->kv_heads = kv_heads; c->max_seq = max_seq; c->head_size = head_size;
    c->layer_elems = max_batch * kv_heads * max_seq * head_size;
    const size_t bytes = layers * c->layer_elems * 2;
    int rc = ellm_device_alloc(device, bytes, &c->k);
    if (rc == ELLM_OK) rc = ellm_device_alloc(device, bytes, &c->v);
    if (rc != ELLM_OK) {
        ellm_device_free(device, c->k);
        delete c;
        return rc;
    }
    *out = c;
    return ELLM_OK;
}

int ellm_kv_cache_destroy(ellm_kv_cache* c) {
    if (!c) return ELLM_OK;
    ellm_device_free(c->device, c->k);
    ellm_device_free(c->device, c->v);
    delete c;
    return ELLM_OK;
}

int ellm_kv_cache_layer(const ellm_kv_cache* c, size_t layer, void** k, void** v, size_t kv_strides[4]) {
    if (!c) return fail(ELLM_ERR_INVALID_ARG, "cache is NULL");
    if (layer >= c->layers) return fail(ELLM_ERR_INVALID_ARG, "layer %zu outside [0, %zu)", layer, c->layers);
    if (k) *k = static_cast<unsigned char*>(c->k) + layer * c->layer_elems * 2;
    if (v) *v = static_cast<unsigned char*>(c->v) + layer * c->layer_elems * 2;
    if (kv_strides) {
        kv_strides[0] = c->kv_heads * c->max_seq * c->head_size;
        kv_strides[1] = c->max_seq * c->head_size;
        kv_strides[2] = c->head_size;
        kv_strides[3] = 1;
    }
    return ELLM_OK;
}

int ellm_kv_append(void* cache, const void* src, const size_t kv_strides[4], size_t max_batch,
                   size_t kv_heads, size_t head_size, size_t max_seq, size_t position_index,
                   const int32_t* positions, size_t position_interval, size_t batch_size, int device,
                   void* stream) {
    if (!cache || !src || !kv_strides) return fail(ELLM_ERR_INVALID_ARG, "cache, src and kv_strides must be non-NULL");
    if (head_size != static_cast<size_t>(ellm::kHeadDim)) return fail(ELLM_ERR_UNSUPPORTED, "head_size %zu: only 128", head_size);
    if (kv_strides[3] != 1) return fail(ELLM_ERR_UNSUPPORTED, "kv_strides[3] must be 1");
    for (int i = 0; i < 3; ++i)
        if (kv_strides[i] % 8 != 0) return fail(ELLM_ERR_INVALID_ARG, "kv_strides[%d] must be a multiple of 8 elements", i);
    if (!aligned16(cache) || !aligned16(src)) return fail(ELLM_ERR_INVALID_ARG, "cache and src must be 16-byte aligned");
    if (batch_size > max_batch) return fail(ELLM_ERR_INVALID_ARG, "batch_size %zu > max_batch %zu", batch_size, max_batch);
    if (!positions && position_index + position_interval > max_seq)
        return fail(ELLM_ERR_INVALID_ARG, "position_index %zu + interval %zu exceeds max_seq %zu", position_index, position_interval, max_seq);
    if (position_interval == 0 || batch_size == 0 || kv_heads == 0) return ELLM_OK;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", device);
    return launch_append(nullptr, static_cast<cudaStream_t>(stream), cache, nullptr, src, nullptr, kv_strides, max_batch,
                         kv_heads, max_seq, position_index, positions, position_interval, batch_size);
}

int ellm_qk_norm_rope_append(const void* q_in, const void* k_in, const void* v_in, void* q_out, void* k_cache,
                             void* v_cache, const float* q_weight, const float* k_weight, const float* rope,
                             size_t rope_rows, const size_t kv_strides[4], size_t max_batch, size_t q_heads,
                             size_t kv_heads, size_t head_size, size_t max_seq, size_t position_index,
                             const int32_t* positions, size_t position_interval, size_t batch_size, float eps,
                             size_t q_in_row_stride, size_t kv_in_row_stride, int device, void* stream) {
    if (!q_in || !k_in || !v_in || !q_out || !k_cache || !v_cache || !rope || !kv_strides)
        return fail(ELLM_ERR_INVALID_ARG, "q_in, k_in, v_in, q_out, k_cache, v_cache, rope and kv_strides must be non-NULL");
    if (head_size != static_cast<size_t>(ellm::kHeadDim)) return fail(ELLM_ERR_UNSUPPORTED, "head_size %zu: only 128", head_size);
    if (kv_strides[3] != 1) return fail(ELLM_ERR_UNSUPPORTED, "kv_strides[3] must be 1");
    for (int i = 0; i < 3; ++i)
        if (kv_strides[i] % 8 != 0 || kv_strides[i] == 0) return fail(ELLM_ERR_INVALID_ARG, "kv_strides[%d] must be a non-zero multiple of 8 elements", i);
    if (!aligned16(q_in) || !aligned16(k_in) || !aligned16(v_in) || !aligned16(q_out) || !aligned16(k_cache) ||
        !aligned16(v_cache) || !aligned16(rope) || !aligned16(q_weight) || !aligned16(k_weight))
        return fail(ELLM_ERR_INVALID_ARG, "buffers must be 16-byte aligned");
    if (q_heads == 0 || kv_heads == 0 || max_batch == 0) return fail(ELLM_ERR_INVALID_ARG, "q_heads, kv_heads, max_batch must be > 0");
    if (batch_size > max_batch) return fail(ELLM_ERR_INVALID_ARG, "batch_size %zu > max_batch %zu", batch_size, max_batch);
    if (!positions && position_index + position_interval > max_seq)
        return fail(ELLM_ERR_INVALID_ARG, "position_index %zu + interval %zu exceeds max_seq %zu", position_index, position_interval, max_seq);
    if (!positions && position_index + position_interval > rope_rows)
        return fail(ELLM_ERR_INVALID_ARG, "the rope table has %zu rows, position %zu is needed", rope_rows, position_index + position_interval - 1);
    if (!(eps >= 0.0f)) return fail(ELLM_ERR_INVALID_ARG, "eps must be >= 0");
    if (position_interval == 0 || batch_size == 0) return ELLM_OK;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", device);
    ellm::NormRopeParams p;
    p.q_in = static_cast<const __nv_bfloat16*>(q_in);
    p.k_in = static_cast<const __nv_bfloat16*>(k_in);
    p.v_in = static_cast<const __nv_bfloat16*>(v_in);
    p.q_out = static_cast<__nv_bfloat16*>(q_out);
    p.k_cache = static_cast<__nv_bfloat16*>(k_cache);
    p.v_cache = static_cast<__nv_bfloat16*>(v_cache);
    p.q_in_stride = static_cast<long long>(q_in_row_stride ? q_in_row_stride : q_heads * head_size);
    p.kv_in_stride = static_cast<long long>(kv_in_row_stride ? kv_in_row_stride : kv_heads * head_size);
    if (p.q_in_stride % 8 != 0 || p.kv_in_stride % 8 != 0 || p.q_in_stride < static_cast<long long>(q_heads * head_size) ||
        p.kv_in_stride < static_cast<long long>(kv_heads * head_size))
        return fail(ELLM_ERR_INVALID_ARG, "input row strides must be multiples of 8 elements and cover a row");
    p.q_weight = q_weight; p.k_weight = k_weight; p.rope = rope;
    p.positions = positions;
    p.position_index = static_cast<long long>(position_index);
    p.s0 = kv_strides[0]; p.s1 = kv_strides[1]; p.s2 = kv_strides[2];
    p.max_seq = static_cast<long long>(max_seq);
    p.rope_rows = static_cast<long long>(rope_rows);
    p.interval = static_cast<int>(position_interval);
    p.batch = static_cast<int>(batch_size);
    p.max_batch = static_cast<int>(max_batch);
    p.q_heads = static_cast<int>(q_heads);
    p.kv_heads = static_cast<int>(kv_heads);
    p.eps = eps;
    const long long warps = static_cast<long long>(position_interval) * batch_size * (q_heads + 2 * kv_heads);
    const long long blocks = (warps + 7) / 8;
    if (blocks > 0x7fffffffll) return fail(ELLM_ERR_UNSUPPORTED, "too many rows for one launch");
    launch_dependent(ellm::qk_norm_rope_append_kernel, static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream), p);
    ELLM_CUDA(cudaGetLastError());
    return ELLM_OK;
}

int ellm_rms_norm(const void* x, void* y, size_t rows, size_t length, float eps, int device, void* stream) {
    if (!x || !y) return fail(ELLM_ERR_INVALID_ARG, "x and y must be non-NULL");
    if (length == 0 || length % 8 != 0) return fail(ELLM_ERR_INVALID_ARG, "length %zu must be a non-zero multiple of 8", length);
    if (!aligned16(x) || !aligned16(y)) return fail(ELLM_ERR_INVALID_ARG, "x and y must be 16-byte aligned");
    if (!(eps >= 0.0f)) return fail(ELLM_ERR_INVALID_ARG, "eps must be >= 0");
    if (rows == 0) return ELLM_OK;
    if (rows > 0x7fffffffull) return fail(ELLM_ERR_UNSUPPORTED, "too many rows for one launch");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", device);
    launch_dependent(ellm::rms_norm_kernel, static_cast<unsigned>(rows), 256, 0, static_cast<cudaStream_t>(stream),
                     static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), static_cast<long long>(rows),
                     static_cast<int>(length), eps);
    ELLM_CUDA(cudaGetLastError());
    return ELLM_OK;
}

static int merge_partials_impl(const float* o_parts, const float* lse_parts, size_t parts, size_t rows,
                               size_t head_size, void* out, bool out_f32, float* lse_out, int device, void* stream) {
    if (!o_parts || !lse_parts || !out) return fail(ELLM_ERR_INVALID_ARG, "o_parts, lse_parts and out must be non-NULL");
    if (head_size != static_cast<size_t>(ellm::kHeadDim)) return fail(ELLM_ERR_UNSUPPORTED, "head_size %zu: only 128", head_size);
    if (parts == 0 || parts > 65535) return fail(ELLM_ERR_INVALID_ARG, "parts %zu out of range", parts);
    if (rows == 0) return ELLM_OK;
    if (!aligned16(o_parts) || !aligned16(out)) return fail(ELLM_ERR_INVALID_ARG, "o_parts and out must be 16-byte aligned");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", device);
    const unsigned blocks = static_cast<unsigned>((rows + 3) / 4);
    if (out_f32)
        ellm::merge_partials_kernel<float><<<blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(
            o_parts, lse_parts, static_cast<int>(parts), static_cast<long long>(rows), static_cast<float*>(out), lse_out);
    else
        ellm::merge_partials_kernel<__nv_bfloat16><<<blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(
            o_parts, lse_parts, static_cast<int>(parts), static_cast<long long>(rows), static_cast<__nv_bfloat16*>(out), lse_out);
    ELLM_CUDA(cudaGetLastError());
    return ELLM_OK;
}

int ellm_attn_merge_partials(const float* o_parts, const float* lse_parts, size_t parts, size_t rows,
                             size_t head_size, void* out, float* lse_out, int device, void* stream) {
    return merge_partials_impl(o_parts, lse_parts, parts, rows, head_size, out, false, lse_out, device, stream);
}

int ellm_attn_merge_partials_f32(const float* o_parts, const float* lse_parts, size_t parts, size_t rows,
                                 size_t head_size, float* out, float* lse_out, int device, void* stream) {
    return merge_partials_impl(o_parts, lse_parts, parts, rows, head_size, out, true, lse_out, device, stream);
}

int ellm_attn_merge_partials_list(const float* const* o_parts, const float* const* lse_parts, size_t parts,
                                  size_t rows, size_t head_size, void* out, int out_is_f32, float* lse_out,
                                  int device, void* stream) {
    if (!o_parts || !lse_parts || !out) return fail(ELLM_ERR_INVALID_ARG, "o_parts, lse_parts and out must be non-NULL");
    if (head_size != static_cast<size_t>(ellm::kHeadDim)) return fail(ELLM_ERR_UNSUPPORTED, "head_size %zu: only 128", head_size);
    if (parts == 0 || parts > static_cast<size_t>(ellm::kMergeListMax))
        return fail(ELLM_ERR_INVALID_ARG, "parts %zu outside [1, %d]", parts, ellm::kMergeListMax);
    if (!aligned16(out)) return fail(ELLM_ERR_INVALID_ARG, "out must be 16-byte aligned");
    ellm::MergeList m{};
    m.parts = static_cast<int>(parts);
    for (size_t i = 0; i < parts; ++i) {
        if (!o_parts[i] || !lse_parts[i]) return fail(ELLM_ERR_INVALID_ARG, "part %zu is NULL", i);
        if (!aligned16(o_parts[i])) return fail(ELLM_ERR_INVALID_ARG, "part %zu must be 16-byte aligned", i);
        m.o[i] = o_parts[i];
        m.lse[i] = lse_parts[i];
    }
    if (rows == 0) return ELLM_OK;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", device);
    const unsigned long long blocks = (rows + 3) / 4;
    if (blocks > 0x7fffffffull) return fail(ELLM_ERR_UNSUPPORTED, "too many rows for one launch");
    if (out_is_f32)
        ellm::merge_partials_list_kernel<float><<<static_cast<unsigned>(blocks), 128, 0, static_cast<cudaStream_t>(stream)>>>(
            m, static_cast<long long>(rows), static_cast<float*>(out), lse_out);
    else
        ellm::merge_partials_list_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 128, 0, static_cast<cudaStream_t>(stream)>>>(
            m, static_cast<long long>(rows), static_cast<__nv_bfloat16*>(out), lse_out);
    ELLM_CUDA(cudaGetLastError());
    return ELLM_OK;
}

// ---- what a host without CUDA bindings needs to run a step asynchronously or as a graph ----
namespace ellm {
__global__ void positions_update_kernel(int32_t* positions, int count, int32_t value, int add) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) positions[i] = add ? positions[i] + value : value;
}
}  // namespace ellm

struct ellm_step_graph {
    int device = 0;
    cudaGraphExec_t exec = nullptr;
    size_t nodes = 0;
};

int ellm_stream_create(int device, void** stream) {
    if (!stream) return fail(ELLM_ERR_INVALID_ARG, "stream is NULL");
    *stream = nullptr;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", device);
    cudaStream_t s = nullptr;
    ELLM_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = s;
    return ELLM_OK;
}

int ellm_stream_destroy(int device, void* stream) {
    if (!stream) return ELLM_OK;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", device);
    ELLM_CUDA(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
    return ELLM_OK;
}

int ellm_stream_synchronize(int device, void* stream) {
    DeviceGuard guard(device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", device);
    ELLM_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    return ELLM_OK;
}

int ellm_positions_set(int32_t* positions, size_t count, int32_t value, int add, int device, void* stream) {
    if (!positions) return fail(ELLM_ERR_INVALID_ARG, "positions is NULL");
    if (count == 0) return ELLM_OK;
    if (count > 0x7fffffffull) return fail(ELLM_ERR_INVALID_ARG, "count too large");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", device);
    const unsigned blocks = static_cast<unsigned>((count + 127) / 128);
    ELLM_CUDA(launch_dependent(ellm::positions_update_kernel, blocks, 128, 0, static_cast<cudaStream_t>(stream), positions,
                               static_cast<int>(count), value, add));
    return ELLM_OK;
}

int ellm_step_graph_begin(int device, void* stream) {
    if (!stream) return fail(ELLM_ERR_INVALID_ARG, "a step can only be captured on a stream made by ellm_stream_create (not the default stream)");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", device);
    ELLM_CUDA(cudaStreamBeginCapture(static_cast<cudaStream_t>(stream), cudaStreamCaptureModeThreadLocal));
    return ELLM_OK;
}

int ellm_step_graph_end(int device, void* stream, ellm_step_graph** out) {
    if (!out) return fail(ELLM_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", device);
    cudaGraph_t graph = nullptr;
    const cudaError_t e = cudaStreamEndCapture(static_cast<cudaStream_t>(stream), &graph);
    if (e != cudaSuccess || !graph) {
        cudaGetLastError();
        return fail(ELLM_ERR_CUDA, "the capture of the step failed: %s (an operator that synchronises or copies "
                    "inside run() cannot be captured: create the operators with async = 1)", cudaGetErrorString(e));
    }
    ellm_step_graph* g = new (std::nothrow) ellm_step_graph();
    if (!g) { cudaGraphDestroy(graph); return fail(ELLM_ERR_NO_MEMORY, "host allocation failed"); }
    g->device = device;
    cudaGraphGetNodes(graph, nullptr, &g->nodes);
    const cudaError_t ei = cudaGraphInstantiate(&g->exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ei != cudaSuccess) {
        delete g;
        cudaGetLastError();
        return fail(ELLM_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(ei));
    }
    *out = g;
    return ELLM_OK;
}

int ellm_step_graph_launch(ellm_step_graph* g, void* stream) {
    if (!g || !g->exec) return fail(ELLM_ERR_INVALID_ARG, "graph is NULL");
    DeviceGuard guard(g->device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", g->device);
    ELLM_CUDA(cudaGraphLaunch(g->exec, static_cast<cudaStream_t>(stream)));
    return ELLM_OK;
}

int ellm_step_graph_nodes(const ellm_step_graph* g, size_t* nodes) {
    if (!g || !nodes) return fail(ELLM_ERR_INVALID_ARG, "graph and nodes must be non-NULL");
    *nodes = g->nodes;
    return ELLM_OK;
}

int ellm_step_graph_destroy(ellm_step_graph* g) {
    if (!g) return ELLM_OK;
    DeviceGuard guard(g->device);
    if (g->exec) cudaGraphExecDestroy(g->exec);
    delete g;
    return ELLM_OK;
}

int ellm_attn_set_option(ellm_attn* h, const char* name, long long value) {
    if (!h || !name) return fail(ELLM_ERR_INVALID_ARG, "handle and name must be non-NULL");
    std::lock_guard<std::mutex> lock(h->mu);
    if (std::strcmp(name, "tc_wait_timeout_ns") == 0) {
        if (value <= 0) return fail(ELLM_ERR_INVALID_ARG, "tc_wait_timeout_ns must be > 0");
        h->tc.wait_timeout_ns = static_cast<unsigned long long>(value);
        return ELLM_OK;
    }
    if (std::strcmp(name, "decode_ctas") == 0) {   // grid of the decode kernel: 1 .. 2 x SMs (the workspace is sized for that)
        if (value < 1 || value > 2 * h->sm_count) return fail(ELLM_ERR_INVALID_ARG, "decode_ctas must be in [1, %d]", 2 * h->sm_count);
        h->dec_ctas = static_cast<int>(value);
        return ELLM_OK;
    }
    if (std::strcmp(name, "decode_early_stream") == 0) {
        h->decode_early = value != 0;
        return ELLM_OK;
    }
    if (std::strcmp(name, "tc_fuse_append") == 0) {
        h->tc.fuse_append = value != 0;
        return ELLM_OK;
    }
    if (std::strcmp(name, "tc_persistent") == 0) {
        h->tc.persistent = value < 0 ? -1 : (value != 0);
        return ELLM_OK;
    }
    if (std::strcmp(name, "tc_debug_skip_kv_item") == 0) {
        h->tc.debug_skip_item = value < 0 ? -1 : static_cast<int>(value);
        return ELLM_OK;
    }
    return fail(ELLM_ERR_INVALID_ARG, "unknown option '%s'", name);
}

int ellm_attn_set_profiling(ellm_attn* h, int on) {
    if (!h) return fail(ELLM_ERR_INVALID_ARG, "handle is NULL");
    std::lock_guard<std::mutex> lock(h->mu);
    h->profiling = on != 0;
    return ELLM_OK;
}

int ellm_attn_kernel_stats(ellm_attn* h, int kernel_id, uint64_t* launches, uint64_t* timed_launches,
                           double* total_ms) {
    if (!h) return fail(ELLM_ERR_INVALID_ARG, "handle is NULL");
    if (kernel_id < 0 || kernel_id >= ELLM_KERNEL_COUNT) return fail(ELLM_ERR_INVALID_ARG, "kernel_id %d unknown", kernel_id);
    DeviceGuard guard(h->d.device);
    std::lock_guard<std::mutex> lock(h->mu);
    auto& pend = h->pending[kernel_id];
    if (!pend.empty()) {
        ELLM_CUDA(cudaStreamSynchronize(h->stream));
        for (auto& pr : pend) {
            float ms = 0.0f;
            if (cudaEventElapsedTime(&ms, pr.first, pr.second) == cudaSuccess) {
                h->total_ms[kernel_id] += ms;
                h->timed[kernel_id]++;
            }
            cudaEventDestroy(pr.first);
            cudaEventDestroy(pr.second);
        }
        pend.clear();
    }
    if (launches) *launches = h->launches[kernel_id];
    if (timed_launches) *timed_launches = h->timed[kernel_id];
    if (total_ms) *total_ms = h->total_ms[kernel_id];
    return ELLM_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Allocation-free decode entry point.
//
// For callers that must not (or cannot) obtain device memory while serving: all
// memory was handed out when the graph was planned, or another allocator in the
// process already owns the whole HBM.  The split-KV partials live in the fixed
// array below instead of a handle's cudaMalloc'd workspace.  Every GPU that loads
// this library holds the array until the process exits.
// ---------------------------------------------------------------------------
namespace {

constexpr size_t kNoAllocPartOBytes = static_cast<size_t>(ELLM_NOALLOC_MAX_SLOTS) * 16 * ellm::kHeadDim * sizeof(float);
constexpr size_t kNoAllocPartLseBytes = static_cast<size_t>(ELLM_NOALLOC_MAX_SLOTS) * 16 * sizeof(float);
constexpr size_t kNoAllocBytes = kNoAllocPartOBytes + kNoAllocPartLseBytes;
static_assert(ELLM_NOALLOC_MAX_BATCH <= ellm::kDecMaxBatch, "the decode kernel's prefix table bounds the batch");

// In host code this name is only a stand-in for the symbol, never a device address:
// the address each device uses is looked up with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

constexpr int kNoAllocMaxDevices = 64;
struct NoAllocDevice {
    unsigned char* scratch = nullptr;  // device address of g_noalloc_scratch on this device
    int sm_count = 0;
    bool ready = false;
};
NoAllocDevice g_noalloc_dev[kNoAllocMaxDevices];
std::mutex g_noalloc_mu;

// Once per device, with that device current.
int noalloc_setup(int device, NoAllocDevice** out) {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    NoAllocDevice& nd = g_noalloc_dev[device];
    if (!nd.ready) {
        void* ptr = nullptr;
        // The look-up can be what loads this library's device image, and with it the array: if
        // another allocator already holds the GPU's memory, this is where that shows.
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e == cudaErrorMemoryAllocation) {
            cudaGetLastError();
            return fail(ELLM_ERR_NO_MEMORY, "no device memory left for the library image and its %zu-byte scratch array on device %d; "
                        "make the first call on a device before another allocator takes its memory", kNoAllocBytes, device);
        }
        ELLM_CUDA(e);
        if (!ptr) return fail(ELLM_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        ELLM_CUDA(cudaDeviceGetAttribute(&nd.sm_count, cudaDevAttrMultiProcessorCount, device));
        int major = 0;
        ELLM_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
        if (major != 10) return fail(ELLM_ERR_UNSUPPORTED, "device %d is not sm_100", device);
        ELLM_CUDA(cudaFuncSetAttribute(ellm::decode_splitkv_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, ellm::kDecSmemBytes));
        ELLM_CUDA(cudaFuncSetAttribute(ellm::decode_splitkv_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, ellm::kDecSmemBytes));
        nd.scratch = static_cast<unsigned char*>(ptr);
        nd.ready = true;
    }
    *out = &nd;
    return ELLM_OK;
}

}  // namespace

extern "C" int ellm_attn_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                        float* lse, const int32_t* positions, size_t position_index,
                                        size_t batch_size, size_t q_heads, size_t kv_heads, size_t head_size,
                                        const size_t kv_strides[4], size_t max_seq, float scale, int device,
                                        void* stream) {
    if (!q || !k_cache || !v_cache || !out || !kv_strides)
        return fail(ELLM_ERR_INVALID_ARG, "q, k_cache, v_cache, out and kv_strides must be non-NULL");
    if (head_size != static_cast<size_t>(ellm::kHeadDim)) return fail(ELLM_ERR_UNSUPPORTED, "head_size %zu: only 128", head_size);
    if (q_heads == 0 || kv_heads == 0 || q_heads % kv_heads != 0)
        return fail(ELLM_ERR_INVALID_ARG, "q_heads %zu must be a non-zero multiple of kv_heads %zu", q_heads, kv_heads);
    if (kv_strides[3] != 1) return fail(ELLM_ERR_UNSUPPORTED, "kv_strides[3] must be 1");
    for (int i = 0; i < 3; ++i)
        if (kv_strides[i] == 0 || kv_strides[i] % 8 != 0)
            return fail(ELLM_ERR_INVALID_ARG, "kv_strides[%d] must be a non-zero multiple of 8 elements", i);
    if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(out))
        return fail(ELLM_ERR_INVALID_ARG, "device buffers must be 16-byte aligned");
    if (lse && (reinterpret_cast<uintptr_t>(lse) & 3u)) return fail(ELLM_ERR_INVALID_ARG, "lse misaligned");
    if (!(scale > 0.0f) || !std::isfinite(scale)) return fail(ELLM_ERR_INVALID_ARG, "scale must be finite and > 0");
    if (max_seq == 0) return fail(ELLM_ERR_INVALID_ARG, "max_seq must be > 0");
    if (!positions && position_index + 1 > max_seq)
        return fail(ELLM_ERR_INVALID_ARG, "position_index %zu is past max_seq %zu", position_index, max_seq);
    if (device < 0 || device >= kNoAllocMaxDevices) return fail(ELLM_ERR_INVALID_ARG, "device %d out of range", device);
    if (batch_size == 0) return ELLM_OK;
    if (batch_size > static_cast<size_t>(ELLM_NOALLOC_MAX_BATCH))
        return fail(ELLM_ERR_UNSUPPORTED, "batch_size %zu exceeds ELLM_NOALLOC_MAX_BATCH %d of the allocation-free entry point",
                    batch_size, ELLM_NOALLOC_MAX_BATCH);
    DeviceGuard guard(device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", device);
    NoAllocDevice* nd = nullptr;
    int rc = noalloc_setup(device, &nd);
    if (rc) return rc;
    const int group = static_cast<int>(q_heads / kv_heads), gtiles = (group + 15) / 16;
    const int num_ctas = 2 * nd->sm_count;
    const size_t slots = static_cast<size_t>(num_ctas) + batch_size * kv_heads * gtiles;
    if (slots > static_cast<size_t>(ELLM_NOALLOC_MAX_SLOTS))
        return fail(ELLM_ERR_UNSUPPORTED,
                    "allocation-free decode needs %zu partial slots (2*%d SMs + batch %zu * kv_heads %zu * head tiles %d) "
                    "but its fixed scratch holds ELLM_NOALLOC_MAX_SLOTS = %d; use a handle (ellm_attn_create) for this size",
                    slots, nd->sm_count, batch_size, kv_heads, gtiles, ELLM_NOALLOC_MAX_SLOTS);
    ellm::DecodeParams p;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
    p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
    p.part_o = reinterpret_cast<float*>(nd->scratch);
    p.part_lse = reinterpret_cast<float*>(nd->scratch + kNoAllocPartOBytes);
    p.positions = positions;
    p.uniform_len = static_cast<long long>(position_index) + 1;
    p.len_cap = static_cast<long long>(max_seq);
    p.key_begin = 0;
    p.s0 = kv_strides[0]; p.s1 = kv_strides[1]; p.s2 = kv_strides[2];
    p.batch = static_cast<int>(batch_size);
    p.q_heads = static_cast<int>(q_heads);
    p.kv_heads = static_cast<int>(kv_heads);
    p.group = group;
    p.gtiles = gtiles;
    p.scale_log2 = scale * ellm::kLog2e;
    p.num_ctas = num_ctas;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (group <= 8) ellm::decode_splitkv_kernel<1><<<num_ctas, ellm::kDecThreads, ellm::kDecSmemBytes, s>>>(p);
    else ellm::decode_splitkv_kernel<2><<<num_ctas, ellm::kDecThreads, ellm::kDecSmemBytes, s>>>(p);
    ELLM_CUDA(cudaGetLastError());
    const unsigned blocks = static_cast<unsigned>(batch_size * q_heads);
    ELLM_CUDA(launch_merge(p, batch_size, blocks, nullptr, out, lse, s, false));
    ELLM_CUDA(cudaGetLastError());
    return ELLM_OK;
}


#ifdef ELLM_TC_TRACE
extern "C" int ellm_debug_read_tc_trace(long long* host, size_t count) {
    return cudaMemcpyFromSymbol(host, ellm::g_tc_trace, count * sizeof(long long)) == cudaSuccess ? 0 : 2;
}
#endif

#ifdef ELLM_CHAIN_TRACE
// reset != 0: forget the records; else copy the record count and (host != NULL) the records, 6 words each
extern "C" int ellm_debug_chain_trace(unsigned long long* host, unsigned* count, int reset) {
    if (reset) {
        const unsigned zero = 0;
        return cudaMemcpyToSymbol(ellm::g_chain_trace_n, &zero, sizeof(zero)) == cudaSuccess ? 0 : 2;
    }
    if (count && cudaMemcpyFromSymbol(count, ellm::g_chain_trace_n, sizeof(unsigned)) != cudaSuccess) return 2;
    if (host && cudaMemcpyFromSymbol(host, ellm::g_chain_trace, sizeof(unsigned long long) * ellm::kChainTraceCap * 6) != cudaSuccess) return 2;
    return 0;
}
#endif

#include "ellm_proj_api.cuh"
