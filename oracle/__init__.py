"""CPU oracle for the eLLM attention path (test infrastructure, not product).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this
package.  `load()` returns a ctypes handle on oracle/_build/libellm_oracle.so,
building it with `make` when it is missing.
"""
from .binding import (  # noqa: F401
    AttnDesc,
    attention_bf16,
    attention_f16_timed,
    assign,
    bf16_bits_to_f32,
    f32_to_bf16_bits,
    flash_attention_f32,
    kv_append_bf16,
    load,
    matmul_nt_bf16,
    merge_partials,
    qk_norm_rope_append_bf16,
    rope_table,
    softmax_attention_f64,
)
