// Row-wise weight-free RMS normalisation, y = x / (sqrt(mean x^2) + eps): the reference's
// rms_norm (src/kernel/generic/rms_norm.rs:6-26; eps is added to the root, not under it).  It is
// the input norm of a decoder layer (src/qwen3_moe/decoder_layer.rs:139-143), i.e. what produces
// the activations the QKV projection reads.  HBM-bound: one read and one write of every row.
// One CTA per row, 8 bf16 per thread per step, fp32 arithmetic.
#pragma once
#include "common.cuh"

namespace ellm {

// 1 / (sqrt(mean x^2) + eps) of one row, computed by a CTA of 256 threads (all must call).  Shared
// with the decode-step projection, which normalises its few input rows itself: the same code, so
// the same sums in the same order and the same bits as this kernel.
__device__ __forceinline__ float block_row_rrms(const uint4* src, int chunks, int length, float eps, float* warp_sums,
                                                float* s_rrms) {
    float ss = 0.0f;
    for (int c = threadIdx.x; c < chunks; c += 256) {
        const uint4 v = src[c];
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float a = __low2float(p[i]), b = __high2float(p[i]);
            ss += a * a + b * b;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < 8; ++w) t += warp_sums[w];
        *s_rrms = 1.0f / (sqrtf(t / static_cast<float>(length)) + eps);
    }
    __syncthreads();
    return *s_rrms;
}

// One 16-byte piece of a row times the row's factor, rounded to bf16.
__device__ __forceinline__ uint4 scale_piece(uint4 v, float rrms) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint4 o;
    uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) po[i] = pack_bf16(__low2float(p[i]) * rrms, __high2float(p[i]) * rrms);
    return o;
}

__global__ void __launch_bounds__(256) rms_norm_kernel(const __nv_bfloat16* x, __nv_bfloat16* y,   // x and y may be the same buffer: no __restrict__
                                                       long long rows, int length, float eps) {
    __shared__ float warp_sums[8];
    __shared__ float s_rrms;
    const long long row = blockIdx.x;
    // a following kernel launched as a programmatic dependent may start its own prologue now;
    // this one, when launched that way itself, waits for the kernel that wrote x
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (row >= rows) return;
    const uint4* src = reinterpret_cast<const uint4*>(x + row * length);
    uint4* dst = reinterpret_cast<uint4*>(y + row * length);
    const int chunks = length / 8;
    const float rrms = block_row_rrms(src, chunks, length, eps, warp_sums, &s_rrms);
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) dst[c] = scale_piece(src[c], rrms);
}

}  // namespace ellm
