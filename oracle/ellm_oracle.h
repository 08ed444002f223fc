// C interface of the CPU oracle (test infrastructure; see ellm_oracle.cpp).
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Arguments of the reference's Attention::new (src/compiler/mul/attention.rs:41-67)
// on host buffers holding bf16 bit patterns, plus the optional LSE output and the
// optional per-sequence positions of the ragged extension.
typedef struct {
    const uint16_t* q;     // [chunk rows, max_batch, q_heads, head_size]
    const uint16_t* k;     // element (b, kvh, pos, c) at b*s0 + kvh*s1 + pos*s2 + c*s3
    const uint16_t* v;
    uint16_t* out;         // same layout as q
    float* lse;            // [chunk rows, max_batch, q_heads] or NULL
    const int32_t* positions;  // [batch] or NULL (then position_index applies to all)
    size_t max_batch, q_heads, kv_heads, head_size;
    size_t kv_strides[4];
    float scale;
} oracle_attn_desc;

float oracle_dot_product_f32(const float* a, const float* b, size_t length);
void oracle_scalar_vector_mul_acc_f32(float scalar1, float* o, float scalar2, const float* v,
                                      size_t length);
void oracle_flash_attention_f32(const float* q, const float* K, const float* V, float* o,
                                float inverse_sqrt_head, size_t length, size_t stride,
                                size_t position, int faithful_scale_defect, float* lse_out);
int oracle_assign(size_t length, size_t num, size_t id, size_t* begin, size_t* end);
void oracle_attention_run_bf16(const oracle_attn_desc* d, size_t position_index,
                               size_t position_interval, size_t batch_size, size_t cpu_num,
                               size_t thread_id);
void oracle_attention_run_threads_bf16(const oracle_attn_desc* d, size_t position_index,
                                       size_t position_interval, size_t batch_size,
                                       size_t threads);
void oracle_kv_append_bf16(uint16_t* cache, const uint16_t* src, const size_t* kv_strides,
                           size_t max_batch, size_t kv_heads, size_t head_size,
                           size_t position_index, size_t position_interval, size_t batch_size,
                           const int32_t* positions);
void oracle_merge_partials_f32(const float* o_parts, const float* lse_parts, size_t parts,
                               size_t rows, size_t head_size, float* o, float* lse);
void oracle_rms_norm_f32(const float* input, float* output, size_t length, float eps);
void oracle_complex_mul_f32(const float* a, const float* b, float* out, size_t length);
void oracle_precompute_freqs_cis(size_t dim, size_t rows, float theta, float* out, int faithful_to_polar);
void oracle_qk_norm_rope_append_bf16(const uint16_t* q_in, const uint16_t* k_in, const uint16_t* v_in,
                                     uint16_t* q_out, uint16_t* k_cache, uint16_t* v_cache,
                                     const float* q_weight, const float* k_weight, const float* rope,
                                     const size_t* kv_strides, size_t max_batch, size_t q_heads,
                                     size_t kv_heads, size_t head_size, size_t position_index,
                                     const int32_t* positions, size_t position_interval, size_t batch_size,
                                     float eps);
void oracle_matmul_nt_bf16(const uint16_t* a, size_t lda, const uint16_t* w_nt, const uint16_t* residual,
                           size_t ldr, uint16_t* out, size_t ldc, size_t m, size_t n, size_t k, size_t threads);
uint16_t oracle_f32_to_bf16(float f);
float oracle_bf16_to_f32(uint16_t h);

// AVX-512-FP16 restatement (ellm_oracle_f16.cpp).  All return 0 / do nothing when the
// CPU lacks avx512fp16; oracle_f16_available() says which.
int oracle_f16_available(void);
float oracle_f16_dot_product(const uint16_t* a, const uint16_t* b, size_t length);
void oracle_f16_scalar_vector_mul_acc(float scalar1, uint16_t* o128, float scalar2,
                                      const uint16_t* v128);
void oracle_f16_flash_attention(const uint16_t* q, const uint16_t* K, const uint16_t* V,
                                uint16_t* o, float inverse_sqrt_head, size_t length,
                                size_t stride, size_t position);
// Same item walk as oracle_attention_run_threads_bf16 but on IEEE half buffers with
// the f16 kernel; returns seconds spent between the first and the last barrier.
double oracle_f16_attention_run_threads(const uint16_t* q, const uint16_t* k, const uint16_t* v,
                                        uint16_t* out, const int32_t* positions,
                                        size_t max_batch, size_t q_heads, size_t kv_heads,
                                        const size_t* kv_strides, float scale,
                                        size_t position_index, size_t position_interval,
                                        size_t batch_size, size_t threads, size_t repeats);

#ifdef __cplusplus
}
#endif
