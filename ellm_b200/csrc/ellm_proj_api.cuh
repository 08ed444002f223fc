// C ABI of include/ellm_proj.h.  Included at the end of ellm_attn_api.cu (one translation unit:
// the error text, the device guard and the status codes are shared with the attention entry points).
#pragma once
#include "../../include/ellm_proj.h"
#include "proj_tcgen05.cuh"

struct ProjHandle {
    int which = 0;                 // 0 = MatMul3, 1 = MatMulAdd
    ellm_matmul3_desc d3{};
    ellm_matmul_add_desc da{};
    int device = 0;
    cudaStream_t stream = nullptr;
    bool async = false;
    ellm::ProjPlan plan;
    CUtensorMap map_w[3];
    CUtensorMap map_a;
    size_t map_a_rows = 0;         // rows map_a was encoded for (0 = none yet)
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
    return ELLM_OK;
}

void proj_common_destroy(ProjHandle* h) {
    DeviceGuard guard(h->device);
    for (auto& pr : h->pending) {
        cudaEventDestroy(pr.first);
        cudaEventDestroy(pr.second);
    }
    cudaFree(h->status_dev);
    if (h->status_host) cudaFreeHost(h->status_host);
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

// A timed-out wait of an earlier enqueue-only run shows up here, at the next call.
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
    p.tiles_m = static_cast<int>((rows + ellm::kPjBM - 1) / ellm::kPjBM);
    p.status = h->status_dev;
    p.wait_timeout_ns = h->plan.wait_timeout_ns;
    const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
    const unsigned grid = static_cast<unsigned>(tiles < h->plan.sm_count ? tiles : h->plan.sm_count);
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (h->profiling) {
        ELLM_CUDA(cudaEventCreate(&e0));
        ELLM_CUDA(cudaEventCreate(&e1));
        ELLM_CUDA(cudaEventRecord(e0, h->stream));
    }
    ellm::proj_tcgen05_kernel<<<grid, ellm::kPjThreads, ellm::kPjSmemBytes, h->stream>>>(h->map_a, h->map_w[0], h->map_w[1],
                                                                                        h->map_w[2], p);
    ELLM_CUDA(cudaGetLastError());
    ++h->launches;
    if (h->profiling) {
        ELLM_CUDA(cudaEventRecord(e1, h->stream));
        h->pending.emplace_back(e0, e1);
    }
    ELLM_CUDA(cudaMemcpyAsync(h->status_host, h->status_dev, sizeof(int), cudaMemcpyDeviceToHost, h->stream));
    if (h->async) return ELLM_OK;
    ELLM_CUDA(cudaStreamSynchronize(h->stream));
    return proj_check_status(h);
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
    if (int st = proj_check_status(h)) return st;
    ellm::ProjParams p{};
    p.mode = ellm::kPjQkv;
    const size_t q_heads = d.b_q_row / 128, kv_heads = d.b_kv_row / 128;
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
    return proj_launch(h, d.hidden, lda, d.col, interval * d.max_batch, p);
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
            if (!ellm::proj_encode_2d(h->plan, &h->map_w[i], w[i], n[i], d->col, d->col, ellm::kPjBN))
                st = fail(ELLM_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled(weight %d) failed", i);
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
    if (st == ELLM_OK && !ellm::proj_encode_2d(h->plan, &h->map_w[0], d->w_nt, d->n_max, d->k_max, d->k_max, ellm::kPjBN))
        st = fail(ELLM_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled(weight) failed");
    if (st != ELLM_OK) {
        proj_common_destroy(h);
        delete h;
        return st;
    }
    h->map_w[1] = h->map_w[0];
    h->map_w[2] = h->map_w[0];
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
    if (int st = proj_check_status(h)) return st;
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
    return proj_launch(h, d.a, lda, d.k_max, position_interval * d.max_batch, p);
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
    if (launches) *launches = h->launches;
    if (timed_launches) *timed_launches = h->timed;
    if (ms) *ms = h->ms;
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
