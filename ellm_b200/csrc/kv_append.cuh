// K4: write the chunk's new K and V rows into the static cache.
//
// The reference keeps K/V in max-shape tensors and writes a chunk's rows at
// [position_begin, ...) (the output_to_kv branch, src/compiler/zip_map/
// complex_zip.rs:92-98; flag src/compiler/mul/matmul.rs:22).  Here the cache is
// [sequence, kv_head, position, head_dim] in HBM (any strides) and this kernel is
// the scatter: pure byte movement, bit-exact.  16 lanes move one 256-byte row.
#pragma once
#include "common.cuh"

namespace ellm {

struct AppendParams {
    const uint4* k_new;  // [interval, max_batch, kv_heads, 128] bf16 viewed as 16-byte chunks
    const uint4* v_new;
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;  // may be nullptr (single-tensor append)
    const int32_t* positions;
    long long position_index;
    long long s0, s1, s2;
    long long max_seq;
    int interval, batch, max_batch, kv_heads;
};

__global__ void __launch_bounds__(256) kv_append_kernel(const AppendParams p) {
    // the kernel that follows (attention, launched as a programmatic dependent) may be set up now
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const long long rows = static_cast<long long>(p.interval) * p.batch * p.kv_heads;
    const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long row = gid >> 4;
    const int chunk = static_cast<int>(gid & 15);
    if (row >= rows) return;
    const int kvh = static_cast<int>(row % p.kv_heads);
    const int b = static_cast<int>((row / p.kv_heads) % p.batch);
    const int h = static_cast<int>(row / (static_cast<long long>(p.kv_heads) * p.batch));
    const long long pos = (p.positions ? static_cast<long long>(p.positions[b]) : p.position_index) + h;
    if (pos < 0 || pos >= p.max_seq) return;  // never write outside the cache
    const long long src = ((static_cast<long long>(h) * p.max_batch + b) * p.kv_heads + kvh) * 16 + chunk;
    const long long dst = b * p.s0 + kvh * p.s1 + pos * p.s2 + chunk * 8;
    *reinterpret_cast<uint4*>(p.k_cache + dst) = p.k_new[src];
    if (p.v_cache) *reinterpret_cast<uint4*>(p.v_cache + dst) = p.v_new[src];
}

}  // namespace ellm
