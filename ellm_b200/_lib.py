"""ctypes loader of libellm_attn.so and the declarations of include/ellm_attn.h.

There is no fallback: if the library is missing and cannot be built, or a call
fails, an exception is raised.
"""
import ctypes as C
import os
import re

from . import build as _build

OK, ERR_INVALID_ARG, ERR_CUDA, ERR_DEVICE_TIMEOUT, ERR_UNSUPPORTED, ERR_NO_MEMORY = range(6)
DTYPE_BF16 = 0
PREFILL_AUTO, PREFILL_TCGEN05, PREFILL_WARP_MMA = 0, 1, 2
KERNEL_KV_APPEND, KERNEL_DECODE_SPLITKV, KERNEL_MERGE, KERNEL_PREFILL_TCGEN05, KERNEL_PREFILL_WARP_MMA = range(5)
NOALLOC_MAX_SLOTS, NOALLOC_MAX_BATCH = 1024, 1024
KERNEL_NAMES = ["kv_append", "decode_splitkv", "merge", "prefill_tcgen05", "prefill_warp_mma"]


class EllmError(RuntimeError):
    def __init__(self, status, text):
        super().__init__(f"ellm_attn status {status}: {text}")
        self.status = status


class AttnDesc(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("out", C.c_void_p),
        ("lse", C.c_void_p), ("k_new", C.c_void_p), ("v_new", C.c_void_p),
        ("max_batch", C.c_size_t), ("q_heads", C.c_size_t), ("kv_heads", C.c_size_t),
        ("head_size", C.c_size_t), ("kv_strides", C.c_size_t * 4), ("max_seq", C.c_size_t),
        ("max_interval", C.c_size_t), ("scale", C.c_float), ("dtype", C.c_int), ("device", C.c_int),
        ("stream", C.c_void_p), ("async_", C.c_int), ("prefill_kernel", C.c_int),
    ]


class MatMul3Desc(C.Structure):
    _fields_ = [
        ("hidden", C.c_void_p), ("hidden_row_stride", C.c_size_t), ("wq_nt", C.c_void_p), ("wk_nt", C.c_void_p),
        ("wv_nt", C.c_void_p), ("q_state", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("kv_strides", C.c_size_t * 4), ("rope", C.c_void_p), ("rope_rows", C.c_size_t),
        ("q_norm_weight", C.c_void_p), ("k_norm_weight", C.c_void_p), ("head_dim", C.c_size_t),
        ("m_row", C.c_size_t), ("col", C.c_size_t), ("b_q_row", C.c_size_t), ("b_kv_row", C.c_size_t),
        ("max_batch", C.c_size_t), ("max_seq", C.c_size_t), ("eps", C.c_float), ("device", C.c_int),
        ("stream", C.c_void_p), ("async_", C.c_int),
        ("input_norm", C.c_int), ("input_norm_eps", C.c_float), ("normed_scratch", C.c_void_p),
    ]


class MatMulAddDesc(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("a_row_stride", C.c_size_t), ("w_nt", C.c_void_p), ("residual", C.c_void_p),
        ("residual_row_stride", C.c_size_t), ("output", C.c_void_p), ("output_row_stride", C.c_size_t),
        ("m_max", C.c_size_t), ("n_max", C.c_size_t), ("k_max", C.c_size_t), ("max_batch", C.c_size_t),
        ("device", C.c_int), ("stream", C.c_void_p), ("async_", C.c_int),
    ]


_lib = None

_SZ, _VP, _I = C.c_size_t, C.c_void_p, C.c_int
_SIGNATURES = {
    "ellm_attn_create": (_I, [C.POINTER(AttnDesc), C.POINTER(_VP)]),
    "ellm_attn_destroy": (_I, [_VP]),
    "ellm_attn_run": (_I, [_VP, _SZ, _SZ, _SZ, _SZ, _SZ]),
    "ellm_attn_run_ragged": (_I, [_VP, _VP, _SZ, _SZ, _SZ, _SZ]),
    "ellm_attn_run_host": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _SZ, _SZ, _SZ]),
    "ellm_device_alloc": (_I, [_I, _SZ, C.POINTER(_VP)]),
    "ellm_device_free": (_I, [_I, _VP]),
    "ellm_kv_cache_create": (_I, [_I, _SZ, _SZ, _SZ, _SZ, _SZ, C.POINTER(_VP)]),
    "ellm_kv_cache_destroy": (_I, [_VP]),
    "ellm_kv_cache_layer": (_I, [_VP, _SZ, C.POINTER(_VP), C.POINTER(_VP), C.POINTER(_SZ)]),
    "ellm_kv_append": (_I, [_VP, _VP, C.POINTER(_SZ), _SZ, _SZ, _SZ, _SZ, _SZ, _VP, _SZ, _SZ, _I, _VP]),
    "ellm_qk_norm_rope_append": (_I, [_VP] * 9 + [_SZ, C.POINTER(_SZ)] + [_SZ] * 6 + [_VP, _SZ, _SZ, C.c_float, _SZ, _SZ, _I, _VP]),
    "ellm_rms_norm": (_I, [_VP, _VP, _SZ, _SZ, C.c_float, _I, _VP]),
    "ellm_attn_merge_partials": (_I, [_VP, _VP, _SZ, _SZ, _SZ, _VP, _VP, _I, _VP]),
    "ellm_attn_merge_partials_f32": (_I, [_VP, _VP, _SZ, _SZ, _SZ, _VP, _VP, _I, _VP]),
    "ellm_attn_run_window": (_I, [_VP, _SZ, _SZ, _SZ, _SZ, _SZ, _VP, _VP]),
    "ellm_attn_run_window_q": (_I, [_VP, _VP, _SZ, _SZ, _SZ, _SZ, _SZ, _VP, _VP]),
    "ellm_attn_merge_partials_list": (_I, [C.POINTER(_VP), C.POINTER(_VP), _SZ, _SZ, _SZ, _VP, _I, _VP, _I, _VP]),
    "ellm_attn_check": (_I, [_VP]),
    "ellm_attn_decode_noalloc": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _SZ, _SZ, _SZ, _SZ, _SZ, C.POINTER(_SZ), _SZ, C.c_float, _I, _VP]),
    "ellm_stream_create": (_I, [_I, C.POINTER(_VP)]),
    "ellm_stream_destroy": (_I, [_I, _VP]),
    "ellm_stream_synchronize": (_I, [_I, _VP]),
    "ellm_positions_set": (_I, [_VP, _SZ, C.c_int32, _I, _I, _VP]),
    "ellm_step_graph_begin": (_I, [_I, _VP]),
    "ellm_step_graph_end": (_I, [_I, _VP, C.POINTER(_VP)]),
    "ellm_step_graph_launch": (_I, [_VP, _VP]),
    "ellm_step_graph_nodes": (_I, [_VP, C.POINTER(_SZ)]),
    "ellm_step_graph_destroy": (_I, [_VP]),
    "ellm_attn_set_option": (_I, [_VP, C.c_char_p, C.c_longlong]),
    "ellm_attn_set_profiling": (_I, [_VP, _I]),
    "ellm_attn_kernel_stats": (_I, [_VP, _I, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_double)]),
    "ellm_matmul3_create": (_I, [C.POINTER(MatMul3Desc), C.POINTER(_VP)]),
    "ellm_matmul3_destroy": (_I, [_VP]),
    "ellm_matmul3_run": (_I, [_VP, _SZ, _SZ, _SZ, _SZ, _SZ]),
    "ellm_matmul3_run_ragged": (_I, [_VP, _VP, _SZ, _SZ, _SZ, _SZ]),
    "ellm_matmul3_set_decode_fusion": (_I, [_VP, _I]),
    "ellm_matmul_add_create": (_I, [C.POINTER(MatMulAddDesc), C.POINTER(_VP)]),
    "ellm_matmul_add_destroy": (_I, [_VP]),
    "ellm_matmul_add_run": (_I, [_VP, _SZ, _SZ, _SZ, _SZ, _SZ]),
    "ellm_matmul_set_profiling": (_I, [_VP, _I, _I]),
    "ellm_matmul_kernel_stats": (_I, [_VP, _I, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_double)]),
    "ellm_matmul_check": (_I, [_VP, _I]),
    "ellm_matmul_set_pairing": (_I, [_VP, _I, _I]),
    "ellm_matmul_debug_skip_load": (_I, [_VP, _I, _I]),
    "ellm_matmul_set_wait_timeout": (_I, [_VP, _I, C.c_ulonglong]),
    "ellm_last_error": (C.c_char_p, []),
    "ellm_status_string": (C.c_char_p, [_I]),
    "ellm_attn_abi_version": (_I, []),
}


def header_symbols():
    """Names of the functions the C headers under include/ declare (parsed from the headers)."""
    names = set()
    for header in ("ellm_attn.h", "ellm_proj.h"):
        with open(os.path.join(_build.INCLUDE, header)) as f:
            text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
        names.update(re.findall(r"\b(ellm_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def load():
    global _lib
    if _lib is not None:
        return _lib
    # ELLM_ATTN_LIB points at an already built library (skips the in-tree build)
    path = os.environ.get("ELLM_ATTN_LIB") or _build.build()
    lib = C.CDLL(path)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def check(status):
    if status != OK:
        raise EllmError(status, load().ellm_last_error().decode())
