"""B200-native attention path for eLLM: the attention operator of the reference's
static graph (causal grouped-query prefill, split-KV decode, KV append into a
static HBM cache) as hand-written sm_100a CUDA behind a C ABI.

The CUDA library is required: importing the operator classes works anywhere,
calling them without libellm_attn.so and a B200 raises.
"""
from ._lib import (  # noqa: F401
    EllmError, PREFILL_AUTO, PREFILL_TCGEN05, PREFILL_WARP_MMA, header_symbols, load,
)
from .attention import (  # noqa: F401
    Attention, decode_noalloc, kv_append, merge_partials, merge_partials_list, qk_norm_rope_append, rms_norm,
)
from .kv_cache import StaticKVCache  # noqa: F401
from .projection import MatMul3, MatMulAdd  # noqa: F401
from .rope import precompute_freqs_cis  # noqa: F401
