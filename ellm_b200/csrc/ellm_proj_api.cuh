// C ABI of include/ellm_proj.h.  Included at the end of ellm_attn_api.cu (one translation unit:
// the error text, the device guard and the status codes are shared with the attention entry points).
#pragma once
#include "../../include/ellm_proj.h"
#include "proj_tcgen05.cuh"
#include "proj_skinny.cuh"

struct ProjHandle {
    int which = 0;                 // 0 = MatMul3, 1 = MatMulAdd
    ellm_matmul3_desc d3{};
    ellm_matmul_add_desc da{};
    int device = 0;
    cudaStream_t stream = nullptr;
    bool async = false;
    ellm::ProjPlan plan;
    CUtensorMap map_w[3];          // boxes of 256 weight rows (one CTA per tile)
    CUtensorMap map_wp[3];         // boxes of 128 weight rows (a CTA pair per tile: each CTA loads half)
    CUtensorMap map_a;
    size_t map_a_rows = 0;         // rows map_a was encoded for (0 = none yet)
    // decode steps (at most 16 rows): the weight-streaming kernel
    struct Skinny {
        const void* w = nullptr;
        size_t n = 0;
        int cols = 0, ctas = 0;
    } sk[3];
    int sk_count = 0;              // 0 = unavailable for this shape, 1 = one matrix, 3 = Wq, Wk, Wv apart
    bool decode_fused = true;      // MatMul3 decode steps: norm + rope + cache write inside the projection kernel
    __nv_bfloat16* qkv_scratch = nullptr;   // MatMul3: the projected rows of a decode step, [16 x (Nq + 2 Nkv)]
    uint64_t skinny_launches = 0;
    int* status_dev = nullptr;
    int* status_host = nullptr;    // pinned mirror
    std::mutex mu;
    bool profiling = false;
    uint64_t launches = 0, timed = 0;
    double ms = 0.0;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pending;
};
struct ellm_matmul3 : ProjHandle {};
struct ellm_matmul_add : ProjHandle {};

namespace {

int proj_check_status(ProjHandle* h);

int proj_common_create(ProjHandle* h, int device, void* stream, int async) {
    h->device = device;
    h->stream = static_cast<cudaStream_t>(stream);
    h->async = async != 0;
    cudaDeviceProp prop;
    ELLM_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return fail(ELLM_ERR_UNSUPPORTED, "device %d is sm_%d%d: this library is built for sm_100a only", device, prop.major, prop.minor);
    ellm::proj_plan_init(h->plan, prop.multiProcessorCount);
    if (!h->plan.ready) return fail(ELLM_ERR_UNSUPPORTED, "tensor-core projection unavailable: %s", h->plan.why);
    if (cudaMalloc(&h->status_dev, sizeof(int)) != cudaSuccess || cudaMallocHost(&h->status_host, sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return fail(ELLM_ERR_NO_MEMORY, "status word allocation failed");
    }
    *h->status_host = 0;
    ELLM_CUDA(cudaMemset(h->status_dev, 0, sizeof(int)));
    static_assert(ellm::kSkSmemMax + 256 + 3072 <= 232448, "shared memory budget: dynamic + static");
    if (cudaFuncSetAttribute(ellm::proj_skinny_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, ellm::kSkSmemMax + 256) != cudaSuccess ||
        cudaFuncSetAttribute(ellm::proj_skinny_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, ellm::kSkSmemMax + 256) != cudaSuccess ||
        cudaFuncSetAttribute(ellm::proj_skinny_kernel<ellm::kSkMaxCols / 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, ellm::kSkSmemMax + 256) != cudaSuccess)
        return fail(ELLM_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(cudaGetLastError()));
    return ELLM_OK;
}

void proj_common_destroy(ProjHandle* h) {
    DeviceGuard guard(h->device);
    for (auto& pr : h->pending) {
        cudaEventDestroy(pr.first);
        cudaEventDestroy(pr.second);
    }
    cudaFree(h->status_dev);
    cudaFree(h->qkv_scratch);
    if (h->status_host) cudaFreeHost(h->status_host);
}

// Plans the weight-streaming kernel for one [n x k] weight: column slices of a multiple of 16 sized
// so that the whole grid is resident at once.  Returns false (and leaves sk.ctas 0) when the shape
// does not fit its shared-memory budget; such handles use the tensor-memory kernel for every run.
bool skinny_plan(ProjHandle* h, ProjHandle::Skinny& sk, const void* w, size_t n, size_t k) {
    sk.ctas = 0;
    const long long blocks16 = static_cast<long long>((n + 15) / 16);
    long long per_cta = (blocks16 + h->plan.sm_count - 1) / h->plan.sm_count;
    if (per_cta * 16 > ellm::kSkMaxCols) per_cta = ellm::kSkMaxCols / 16;
    const int cols = static_cast<int>(per_cta * 16);
    if (ellm::skinny_pick_pass_chunks(static_cast<int>(k / 8), cols, 1) < 0) return false;   // not even one row fits
    sk.w = w;
    sk.n = n;
    sk.cols = cols;
    sk.ctas = static_cast<int>((n + cols - 1) / cols);
    return true;
}

// One launch of the weight-streaming kernel, allowed to start while the stream's previous kernel
// is still running: its weight loads do not depend on that kernel, its activations are read after
// a device-side wait for it.
// fused != nullptr: the head epilogue (its fields of SkinnyParams filled in), 16 columns per CTA, clusters of 8.
int skinny_launch(ProjHandle* h, const ProjHandle::Skinny& sk, const void* a, size_t lda, size_t k, size_t rows,
                  size_t batch, size_t max_batch, void* c, size_t ldc, const void* residual, size_t ldr,
                  float input_norm_eps = -1.0f, const ellm::SkinnyParams* fused = nullptr) {
    ellm::SkinnyParams p{};
    if (fused) p = *fused;
    const int cols = fused ? 16 : sk.cols;
    p.a = static_cast<const __nv_bfloat16*>(a);
    p.lda = static_cast<long long>(lda);
    p.m_rows = static_cast<int>(rows);
    p.batch = static_cast<int>(batch);
    p.max_batch = static_cast<int>(max_batch);
    p.w = static_cast<const __nv_bfloat16*>(sk.w);
    p.k_chunks = static_cast<int>(k / 8);
    p.cols = cols;
    p.n_cols = static_cast<int>(sk.n);
    // the slice takes what the activation rows of this run leave of the shared memory
    p.pass_chunks = ellm::skinny_pick_pass_chunks(p.k_chunks, cols, p.m_rows);
    if (p.pass_chunks < 0) return fail(ELLM_ERR_UNSUPPORTED, "no shared-memory plan for %zu rows of %zu", rows, k);
    p.c = static_cast<__nv_bfloat16*>(c);
    p.ldc = static_cast<long long>(ldc);
    p.residual = static_cast<const __nv_bfloat16*>(residual);
    p.ldr = static_cast<long long>(ldr);
    p.input_norm_eps = input_norm_eps;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(fused ? sk.n / 16 : sk.ctas));
    cfg.blockDim = dim3(ellm::kSkThreads);
    cfg.dynamicSmemBytes = static_cast<size_t>(ellm::skinny_smem_bytes(p.k_chunks, cols, p.pass_chunks, p.m_rows));
    cfg.stream = h->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;   // the 8 CTAs of a head
    attr[1].val.clusterDim.x = 8;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = fused ? 2 : 1;
    const cudaError_t e = cols == 16 && rows > 8 ? cudaLaunchKernelEx(&cfg, ellm::proj_skinny_kernel<1, true>, p)
                          : cols == 16 ? cudaLaunchKernelEx(&cfg, ellm::proj_skinny_kernel<1>, p)
                                     : cudaLaunchKernelEx(&cfg, ellm::proj_skinny_kernel<ellm::kSkMaxCols / 16>, p);
    if (e != cudaSuccess) return fail(ELLM_ERR_CUDA, "projection launch failed: %s", cudaGetErrorString(e));
    ++h->skinny_launches;
    return ELLM_OK;
}

// Tail of a run.  A synchronous handle waits for the stream and reads the status word; an
// enqueue-only handle adds nothing to the stream (its caller may be capturing a graph of many
// small steps) and learns of a timed-out wait from ellm_matmul_check().
int proj_finish(ProjHandle* h) {
    if (h->async) return ELLM_OK;
    ELLM_CUDA(cudaMemcpyAsync(h->status_host, h->status_dev, sizeof(int), cudaMemcpyDeviceToHost, h->stream));
    ELLM_CUDA(cudaStreamSynchronize(h->stream));
    return proj_check_status(h);
}

void proj_collect(ProjHandle* h) {  // folds finished event pairs into the totals
    size_t keep = 0;
    for (auto& pr : h->pending) {
        float t = 0.f;
        if (cudaEventQuery(pr.second) == cudaSuccess && cudaEventElapsedTime(&t, pr.first, pr.second) == cudaSuccess) {
            h->ms += t;
            ++h->timed;
            cudaEventDestroy(pr.first);
            cudaEventDestroy(pr.second);
        } else {
            cudaGetLastError();
            h->pending[keep++] = pr;
        }
    }
    h->pending.resize(keep);
}

int proj_check_status(ProjHandle* h) {
    if (h->status_host && *h->status_host != 0) {
        const int code = *h->status_host;
        *h->status_host = 0;
        cudaMemsetAsync(h->status_dev, 0, sizeof(int), h->stream);
        return fail(ELLM_ERR_DEVICE_TIMEOUT, "a bounded device-side wait ran out (code %d)", code);
    }
    return ELLM_OK;
}

int proj_launch(ProjHandle* h, const void* a, size_t lda, size_t k, size_t rows, ellm::ProjParams& p) {
    if (h->map_a_rows != rows) {
        if (!ellm::proj_encode_2d(h->plan, &h->map_a, a, rows, k, lda, ellm::kPjBM))
            return fail(ELLM_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled(A) failed");
        h->map_a_rows = rows;
    }
    p.m_rows = static_cast<int>(rows);
    p.k_blocks = static_cast<int>(k / ellm::kPjBK);
    p.status = h->status_dev;
    p.wait_timeout_ns = h->plan.wait_timeout_ns;
    p.debug_skip_load = h->plan.debug_skip_load;
    // CTA pairs on 256 x 256 tiles when every pair gets at least four of them (a pair loads a third
    // less per CTA from L2; with few tiles the finer 128-row tiles balance better)
    const long long tiles256 = static_cast<long long>((rows + 255) / 256) * p.tiles_n;
    const int pairs = h->plan.sm_count / 2;
    const bool pair = h->plan.pairing == 1 ? rows > 128 : (h->plan.pairing == -1 && tiles256 >= 4ll * pairs);
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (h->profiling) {
        ELLM_CUDA(cudaEventCreate(&e0));
        ELLM_CUDA(cudaEventCreate(&e1));
        ELLM_CUDA(cudaEventRecord(e0, h->stream));
    }
    if (pair) {
        p.tiles_m = static_cast<int>((rows + 255) / 256);
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(static_cast<unsigned>(2 * (tiles256 < pairs ? tiles256 : pairs)));
        cfg.blockDim = dim3(ellm::kPjThreads);
        cfg.dynamicSmemBytes = ellm::kPjSmemBytes;
        cfg.stream = h->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, ellm::proj_tcgen05_kernel<true>, h->map_a, h->map_wp[0], h->map_wp[1],
                                                 h->map_wp[2], p);
        if (e != cudaSuccess) return fail(ELLM_ERR_CUDA, "projection launch failed: %s", cudaGetErrorString(e));
    } else {
        p.tiles_m = static_cast<int>((rows + ellm::kPjBM - 1) / ellm::kPjBM);
        const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
        const unsigned grid = static_cast<unsigned>(tiles < h->plan.sm_count ? tiles : h->plan.sm_count);
        ellm::proj_tcgen05_kernel<false><<<grid, ellm::kPjThreads, ellm::kPjSmemBytes, h->stream>>>(h->map_a, h->map_w[0], h->map_w[1],
                                                                                                   h->map_w[2], p);
        ELLM_CUDA(cudaGetLastError());
    }
    ++h->launches;
    if (h->profiling) {
        ELLM_CUDA(cudaEventRecord(e1, h->stream));
        h->pending.emplace_back(e0, e1);
    }
    return proj_finish(h);
}

int matmul3_run_impl(ellm_matmul3* h, const int32_t* positions, size_t position_index, size_t interval, size_t batch,
                     size_t thread_id) {
    if (!h) return fail(ELLM_ERR_INVALID_ARG, "handle is NULL");
    if (thread_id != 0) return ELLM_OK;
    const ellm_matmul3_desc& d = h->d3;
    if (batch > d.max_batch) return fail(ELLM_ERR_INVALID_ARG, "batch_size %zu > max_batch %zu", batch, d.max_batch);
    if (interval * d.max_batch > d.m_row) return fail(ELLM_ERR_INVALID_ARG, "position_interval %zu x max_batch %zu exceeds m_row %zu", interval, d.max_batch, d.m_row);
    if (!positions && position_index + interval > d.max_seq)
        return fail(ELLM_ERR_INVALID_ARG, "position_index %zu + interval %zu exceeds max_seq %zu", position_index, interval, d.max_seq);
    if (!positions && position_index + interval > d.rope_rows)
        return fail(ELLM_ERR_INVALID_ARG, "the rope table has %zu rows, position %zu is needed", d.rope_rows, position_index + interval - 1);
    if (interval == 0 || batch == 0) return ELLM_OK;
    std::lock_guard<std::mutex> lock(h->mu);
    DeviceGuard guard(h->device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", h->device);
    const size_t q_heads = d.b_q_row / 128, kv_heads = d.b_kv_row / 128;
    const size_t rows = interval * d.max_batch;
    if (rows <= static_cast<size_t>(ellm::kSkRows) && h->sk_count > 0) {
        // decode step: stream the weights once, then norm + rope + cache write on the projected rows
        const size_t lda = d.hidden_row_stride ? d.hidden_row_stride : d.col;
        const size_t ldq = d.b_q_row + 2 * d.b_kv_row;
        if (h->decode_fused) {
            // one kernel per weight matrix: projection, head norm, rotation, Q store and cache write
            ellm::SkinnyParams f{};
            f.q_heads = static_cast<int>(q_heads);
            f.q_out = static_cast<__nv_bfloat16*>(d.q_state);
            f.k_cache = static_cast<__nv_bfloat16*>(d.k_cache);
            f.v_cache = static_cast<__nv_bfloat16*>(d.v_cache);
            f.q_norm_weight = d.q_norm_weight;
            f.k_norm_weight = d.k_norm_weight;
            f.rope = d.rope;
            f.positions = positions;
            f.position_index = static_cast<long long>(position_index);
            f.s0 = d.kv_strides[0]; f.s1 = d.kv_strides[1]; f.s2 = d.kv_strides[2];
            f.max_seq = static_cast<long long>(d.max_seq);
            f.rope_rows = static_cast<long long>(d.rope_rows);
            f.eps = d.eps;
            for (int i = 0; i < h->sk_count; ++i) {
                f.heads = static_cast<int>(h->sk[i].n / 128);
                f.mat_q_heads = h->sk_count == 1 ? static_cast<int>(q_heads) : (i == 0 ? f.heads : 0);
                f.mat_k_heads = h->sk_count == 1 ? static_cast<int>(kv_heads) : (i == 1 ? f.heads : 0);
                if (int st = skinny_launch(h, h->sk[i], d.hidden, lda, d.col, rows, batch, d.max_batch, nullptr, 0, nullptr, 0,
                                           d.input_norm ? d.input_norm_eps : -1.0f, &f))
                    return st;
            }
            return proj_finish(h);
        }
        size_t col0 = 0;
        for (int i = 0; i < h->sk_count; ++i) {
            if (int st = skinny_launch(h, h->sk[i], d.hidden, lda, d.col, rows, batch, d.max_batch, h->qkv_scratch + col0, ldq,
                                       nullptr, 0, d.input_norm ? d.input_norm_eps : -1.0f))
                return st;
            col0 += h->sk[i].n;
        }
        if (int st = ellm_qk_norm_rope_append(h->qkv_scratch, h->qkv_scratch + d.b_q_row, h->qkv_scratch + d.b_q_row + d.b_kv_row,
                                              d.q_state, d.k_cache, d.v_cache, d.q_norm_weight, d.k_norm_weight, d.rope,
                                              d.rope_rows, d.kv_strides, d.max_batch, q_heads, kv_heads, 128, d.max_seq,
                                              position_index, positions, interval, batch, d.eps, ldq, ldq, h->device, h->stream))
            return st;
        return proj_finish(h);
    }
    ellm::ProjParams p{};
    p.mode = ellm::kPjQkv;
    p.tiles_q = static_cast<int>((q_heads + 1) / 2);
    p.tiles_kv = static_cast<int>((kv_heads + 1) / 2);
    p.tiles_n = p.tiles_q + 2 * p.tiles_kv;
    p.batch = static_cast<int>(batch);
    p.max_batch = static_cast<int>(d.max_batch);
    p.q_out = static_cast<__nv_bfloat16*>(d.q_state);
    p.k_cache = static_cast<__nv_bfloat16*>(d.k_cache);
    p.v_cache = static_cast<__nv_bfloat16*>(d.v_cache);
    p.q_weight = d.q_norm_weight;
    p.k_weight = d.k_norm_weight;
    p.rope = d.rope;
    p.positions = positions;
    p.position_index = static_cast<long long>(position_index);
    p.s0 = d.kv_strides[0]; p.s1 = d.kv_strides[1]; p.s2 = d.kv_strides[2];
    p.max_seq = static_cast<long long>(d.max_seq);
    p.rope_rows = static_cast<long long>(d.rope_rows);
    p.q_heads = static_cast<int>(q_heads);
    p.kv_heads = static_cast<int>(kv_heads);
    p.eps = d.eps;
    const size_t lda = d.hidden_row_stride ? d.hidden_row_stride : d.col;
    if (d.input_norm) {
        if (lda != d.col) return fail(ELLM_ERR_UNSUPPORTED, "input_norm needs contiguous rows of hidden");
        if (int st = ellm_rms_norm(d.hidden, d.normed_scratch, rows, d.col, d.input_norm_eps, h->device, h->stream)) return st;
        return proj_launch(h, d.normed_scratch, d.col, d.col, rows, p);
    }
    return proj_launch(h, d.hidden, lda, d.col, rows, p);
}

bool proj_stride_ok(size_t stride, size_t width) { return stride % 8 == 0 && stride >= width; }

}  // namespace

extern "C" {

int ellm_matmul3_create(const ellm_matmul3_desc* d, ellm_matmul3** out) {
    if (!d || !out) return fail(ELLM_ERR_INVALID_ARG, "desc and out must be non-NULL");
    *out = nullptr;
    if (!d->hidden || !d->wq_nt || !d->wk_nt || !d->wv_nt || !d->q_state || !d->k_cache || !d->v_cache || !d->rope)
        return fail(ELLM_ERR_INVALID_ARG, "hidden, wq_nt, wk_nt, wv_nt, q_state, k_cache, v_cache and rope must be non-NULL");
    if (d->head_dim != 128) return fail(ELLM_ERR_UNSUPPORTED, "head_dim %zu: only 128", d->head_dim);
    if (d->col == 0 || d->col % 64 != 0) return fail(ELLM_ERR_UNSUPPORTED, "col (K) %zu must be a non-zero multiple of 64", d->col);
    if (d->b_q_row == 0 || d->b_q_row % 128 != 0 || d->b_kv_row == 0 || d->b_kv_row % 128 != 0)
        return fail(ELLM_ERR_INVALID_ARG, "b_q_row %zu and b_kv_row %zu must be non-zero multiples of head_dim", d->b_q_row, d->b_kv_row);
    if ((d->b_q_row / 128) % (d->b_kv_row / 128) != 0) return fail(ELLM_ERR_INVALID_ARG, "query heads must be a multiple of KV heads");
    if (d->max_batch == 0 || d->m_row == 0 || d->m_row % d->max_batch != 0)
        return fail(ELLM_ERR_INVALID_ARG, "m_row %zu must be a non-zero multiple of max_batch %zu", d->m_row, d->max_batch);
    if (d->m_row > 0x7fffff00ull) return fail(ELLM_ERR_UNSUPPORTED, "m_row %zu too large", d->m_row);
    const size_t lda = d->hidden_row_stride ? d->hidden_row_stride : d->col;
    if (!proj_stride_ok(lda, d->col)) return fail(ELLM_ERR_INVALID_ARG, "hidden_row_stride must be a multiple of 8 elements and cover a row");
    if (d->kv_strides[3] != 1) return fail(ELLM_ERR_UNSUPPORTED, "kv_strides[3] must be 1");
    for (int i = 0; i < 3; ++i)
        if (d->kv_strides[i] % 8 != 0 || d->kv_strides[i] == 0) return fail(ELLM_ERR_INVALID_ARG, "kv_strides[%d] must be a non-zero multiple of 8 elements", i);
    if (!aligned16(d->hidden) || !aligned16(d->wq_nt) || !aligned16(d->wk_nt) || !aligned16(d->wv_nt) || !aligned16(d->q_state) ||
        !aligned16(d->k_cache) || !aligned16(d->v_cache) || !aligned16(d->rope) || !aligned16(d->q_norm_weight) || !aligned16(d->k_norm_weight))
        return fail(ELLM_ERR_INVALID_ARG, "buffers must be 16-byte aligned");
    if (!(d->eps >= 0.0f)) return fail(ELLM_ERR_INVALID_ARG, "eps must be >= 0");
    if (d->max_seq == 0 || d->rope_rows == 0) return fail(ELLM_ERR_INVALID_ARG, "max_seq and rope_rows must be > 0");
    if (d->input_norm && (!(d->input_norm_eps >= 0.0f) || !d->normed_scratch || !aligned16(d->normed_scratch)))
        return fail(ELLM_ERR_INVALID_ARG, "input_norm needs input_norm_eps >= 0 and a 16-byte aligned normed_scratch");
    DeviceGuard guard(d->device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", d->device);
    ellm_matmul3* h = new (std::nothrow) ellm_matmul3();
    if (!h) return fail(ELLM_ERR_NO_MEMORY, "out of host memory");
    h->which = 0;
    h->d3 = *d;
    int st = proj_common_create(h, d->device, d->stream, d->async);
    if (st == ELLM_OK) {
        const void* w[3] = {d->wq_nt, d->wk_nt, d->wv_nt};
        const size_t n[3] = {d->b_q_row, d->b_kv_row, d->b_kv_row};
        for (int i = 0; i < 3 && st == ELLM_OK; ++i)
            if (!ellm::proj_encode_2d(h->plan, &h->map_w[i], w[i], n[i], d->col, d->col, ellm::kPjBN) ||
                !ellm::proj_encode_2d(h->plan, &h->map_wp[i], w[i], n[i], d->col, d->col, ellm::kPjBN / 2))
                st = fail(ELLM_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled(weight %d) failed", i);
    }
    if (st == ELLM_OK) {
        // decode path: one matrix when Wq, Wk, Wv lie back to back, else one launch per weight
        const char* wq = static_cast<const char*>(d->wq_nt);
        const bool contiguous = static_cast<const char*>(d->wk_nt) == wq + d->b_q_row * d->col * 2 &&
                                static_cast<const char*>(d->wv_nt) == wq + (d->b_q_row + d->b_kv_row) * d->col * 2;
        bool ok;
        if (contiguous) {
            ok = skinny_plan(h, h->sk[0], d->wq_nt, d->b_q_row + 2 * d->b_kv_row, d->col);
            h->sk_count = ok ? 1 : 0;
        } else {
            ok = skinny_plan(h, h->sk[0], d->wq_nt, d->b_q_row, d->col) && skinny_plan(h, h->sk[1], d->wk_nt, d->b_kv_row, d->col) &&
                 skinny_plan(h, h->sk[2], d->wv_nt, d->b_kv_row, d->col);
            h->sk_count = ok ? 3 : 0;
        }
        if (ok && cudaMalloc(&h->qkv_scratch, ellm::kSkRows * (d->b_q_row + 2 * d->b_kv_row) * 2) != cudaSuccess) {
            cudaGetLastError();
            st = fail(ELLM_ERR_NO_MEMORY, "scratch allocation failed");
        }
    }
    if (st != ELLM_OK) {
        proj_common_destroy(h);
        delete h;
        return st;
    }
    *out = h;
    return ELLM_OK;
}

int ellm_matmul3_destroy(ellm_matmul3* h) {
    if (!h) return ELLM_OK;
    proj_common_destroy(h);
    delete h;
    return ELLM_OK;
}

int ellm_matmul3_run(ellm_matmul3* h, size_t position_index, size_t position_interval, size_t batch_size, size_t cpu_num,
                     size_t thread_id) {
    (void)cpu_num;
    return matmul3_run_impl(h, nullptr, position_index, position_interval, batch_size, thread_id);
}

int ellm_matmul3_run_ragged(ellm_matmul3* h, const int32_t* positions, size_t position_interval, size_t batch_size,
                            size_t cpu_num, size_t thread_id) {
    (void)cpu_num;
    if (!positions) return fail(ELLM_ERR_INVALID_ARG, "positions is NULL");
    return matmul3_run_impl(h, positions, 0, position_interval, batch_size, thread_id);
}

int ellm_matmul_add_create(const ellm_matmul_add_desc* d, ellm_matmul_add** out) {
    if (!d || !out) return fail(ELLM_ERR_INVALID_ARG, "desc and out must be non-NULL");
    *out = nullptr;
    if (!d->a || !d->w_nt || !d->output) return fail(ELLM_ERR_INVALID_ARG, "a, w_nt and output must be non-NULL");
    if (d->k_max == 0 || d->k_max % 64 != 0) return fail(ELLM_ERR_UNSUPPORTED, "k_max %zu must be a non-zero multiple of 64", d->k_max);
    if (d->n_max == 0 || d->n_max % 8 != 0) return fail(ELLM_ERR_UNSUPPORTED, "n_max %zu must be a non-zero multiple of 8", d->n_max);
    if (d->max_batch == 0 || d->m_max == 0 || d->m_max % d->max_batch != 0)
        return fail(ELLM_ERR_INVALID_ARG, "m_max %zu must be a non-zero multiple of max_batch %zu", d->m_max, d->max_batch);
    if (d->m_max > 0x7fffff00ull || d->n_max > 0x7fffff00ull) return fail(ELLM_ERR_UNSUPPORTED, "matrix too large");
    const size_t lda = d->a_row_stride ? d->a_row_stride : d->k_max;
    const size_t ldr = d->residual_row_stride ? d->residual_row_stride : d->n_max;
    const size_t ldc = d->output_row_stride ? d->output_row_stride : d->n_max;
    if (!proj_stride_ok(lda, d->k_max) || !proj_stride_ok(ldr, d->n_max) || !proj_stride_ok(ldc, d->n_max))
        return fail(ELLM_ERR_INVALID_ARG, "row strides must be multiples of 8 elements and cover a row");
    if (!aligned16(d->a) || !aligned16(d->w_nt) || !aligned16(d->residual) || !aligned16(d->output))
        return fail(ELLM_ERR_INVALID_ARG, "buffers must be 16-byte aligned");
    DeviceGuard guard(d->device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", d->device);
    ellm_matmul_add* h = new (std::nothrow) ellm_matmul_add();
    if (!h) return fail(ELLM_ERR_NO_MEMORY, "out of host memory");
    h->which = 1;
    h->da = *d;
    int st = proj_common_create(h, d->device, d->stream, d->async);
    if (st == ELLM_OK && (!ellm::proj_encode_2d(h->plan, &h->map_w[0], d->w_nt, d->n_max, d->k_max, d->k_max, ellm::kPjBN) ||
                          !ellm::proj_encode_2d(h->plan, &h->map_wp[0], d->w_nt, d->n_max, d->k_max, d->k_max, ellm::kPjBN / 2)))
        st = fail(ELLM_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled(weight) failed");
    if (st != ELLM_OK) {
        proj_common_destroy(h);
        delete h;
        return st;
    }
    h->map_w[1] = h->map_w[2] = h->map_w[0];
    h->map_wp[1] = h->map_wp[2] = h->map_wp[0];
    h->sk_count = skinny_plan(h, h->sk[0], d->w_nt, d->n_max, d->k_max) ? 1 : 0;
    *out = h;
    return ELLM_OK;
}

int ellm_matmul_add_destroy(ellm_matmul_add* h) {
    if (!h) return ELLM_OK;
    proj_common_destroy(h);
    delete h;
    return ELLM_OK;
}

int ellm_matmul_add_run(ellm_matmul_add* h, size_t position_index, size_t position_interval, size_t batch_size,
                        size_t cpu_num, size_t thread_id) {
    (void)position_index;
    (void)cpu_num;
    if (!h) return fail(ELLM_ERR_INVALID_ARG, "handle is NULL");
    if (thread_id != 0) return ELLM_OK;
    const ellm_matmul_add_desc& d = h->da;
    if (batch_size > d.max_batch) return fail(ELLM_ERR_INVALID_ARG, "batch_size %zu > max_batch %zu", batch_size, d.max_batch);
    if (position_interval * d.max_batch > d.m_max)
        return fail(ELLM_ERR_INVALID_ARG, "position_interval %zu x max_batch %zu exceeds m_max %zu", position_interval, d.max_batch, d.m_max);
    if (position_interval == 0 || batch_size == 0) return ELLM_OK;
    std::lock_guard<std::mutex> lock(h->mu);
    DeviceGuard guard(h->device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", h->device);
    const size_t rows = position_interval * d.max_batch;
    if (rows <= static_cast<size_t>(ellm::kSkRows) && h->sk_count > 0) {
        if (int st = skinny_launch(h, h->sk[0], d.a, d.a_row_stride ? d.a_row_stride : d.k_max, d.k_max, rows, batch_size,
                                   d.max_batch, d.output, d.output_row_stride ? d.output_row_stride : d.n_max, d.residual,
                                   d.residual_row_stride ? d.residual_row_stride : d.n_max))
            return st;
        return proj_finish(h);
    }
    ellm::ProjParams p{};
    p.mode = ellm::kPjPlain;
    p.tiles_n = static_cast<int>((d.n_max + ellm::kPjBN - 1) / ellm::kPjBN);
    p.batch = static_cast<int>(batch_size);
    p.max_batch = static_cast<int>(d.max_batch);
    p.c = static_cast<__nv_bfloat16*>(d.output);
    p.residual = static_cast<const __nv_bfloat16*>(d.residual);
    p.ldc = static_cast<long long>(d.output_row_stride ? d.output_row_stride : d.n_max);
    p.ldr = static_cast<long long>(d.residual_row_stride ? d.residual_row_stride : d.n_max);
    p.n_cols = static_cast<int>(d.n_max);
    const size_t lda = d.a_row_stride ? d.a_row_stride : d.k_max;
    return proj_launch(h, d.a, lda, d.k_max, rows, p);
}

static ProjHandle* proj_cast(void* handle, int which) {
    ProjHandle* h = static_cast<ProjHandle*>(handle);
    return (h && h->which == which) ? h : nullptr;
}

int ellm_matmul_set_profiling(void* handle, int which, int on) {
    ProjHandle* h = proj_cast(handle, which);
    if (!h) return fail(ELLM_ERR_INVALID_ARG, "handle is NULL or not of kind %d", which);
    std::lock_guard<std::mutex> lock(h->mu);
    h->profiling = on != 0;
    return ELLM_OK;
}

int ellm_matmul_kernel_stats(void* handle, int which, uint64_t* launches, uint64_t* timed_launches, double* ms) {
    ProjHandle* h = proj_cast(handle, which);
    if (!h) return fail(ELLM_ERR_INVALID_ARG, "handle is NULL or not of kind %d", which);
    std::lock_guard<std::mutex> lock(h->mu);
    DeviceGuard guard(h->device);
    proj_collect(h);
    if (launches) *launches = h->launches + h->skinny_launches;
    if (timed_launches) *timed_launches = h->timed;
    if (ms) *ms = h->ms;
    return ELLM_OK;
}

int ellm_matmul_check(void* handle, int which) {
    ProjHandle* h = proj_cast(handle, which);
    if (!h) return fail(ELLM_ERR_INVALID_ARG, "handle is NULL or not of kind %d", which);
    std::lock_guard<std::mutex> lock(h->mu);
    DeviceGuard guard(h->device);
    if (!guard.ok) return fail(ELLM_ERR_CUDA, "cannot select device %d", h->device);
    ELLM_CUDA(cudaMemcpyAsync(h->status_host, h->status_dev, sizeof(int), cudaMemcpyDeviceToHost, h->stream));
    ELLM_CUDA(cudaStreamSynchronize(h->stream));
    return proj_check_status(h);
}

int ellm_matmul3_set_decode_fusion(ellm_matmul3* h, int on) {
    if (!h) return fail(ELLM_ERR_INVALID_ARG, "handle is NULL");
    std::lock_guard<std::mutex> lock(h->mu);
    h->decode_fused = on != 0;
    return ELLM_OK;
}

int ellm_matmul_set_pairing(void* handle, int which, int mode) {
    ProjHandle* h = proj_cast(handle, which);
    if (!h) return fail(ELLM_ERR_INVALID_ARG, "handle is NULL or not of kind %d", which);
    if (mode < -1 || mode > 1) return fail(ELLM_ERR_INVALID_ARG, "mode must be -1, 0 or 1");
    std::lock_guard<std::mutex> lock(h->mu);
    h->plan.pairing = mode;
    return ELLM_OK;
}

int ellm_matmul_debug_skip_load(void* handle, int which, int item) {
    ProjHandle* h = proj_cast(handle, which);
    if (!h) return fail(ELLM_ERR_INVALID_ARG, "handle is NULL or not of kind %d", which);
    std::lock_guard<std::mutex> lock(h->mu);
    h->plan.debug_skip_load = item < 0 ? -1 : item;
    return ELLM_OK;
}

int ellm_matmul_set_wait_timeout(void* handle, int which, unsigned long long ns) {
    ProjHandle* h = proj_cast(handle, which);
    if (!h) return fail(ELLM_ERR_INVALID_ARG, "handle is NULL or not of kind %d", which);
    if (ns == 0) return fail(ELLM_ERR_INVALID_ARG, "timeout must be > 0");
    std::lock_guard<std::mutex> lock(h->mu);
    h->plan.wait_timeout_ns = ns;
    return ELLM_OK;
}

}  // extern "C"
