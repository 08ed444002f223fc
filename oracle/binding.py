"""ctypes binding of the CPU oracle plus an independent float64 cross-check.

Test infrastructure: see ellm_oracle.cpp for what each entry point restates.
Buffers are numpy arrays; bf16 / f16 data travel as uint16 bit patterns.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libellm_oracle.so")
_lib = None


class AttnDesc(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("lse", C.c_void_p), ("positions", C.c_void_p),
        ("max_batch", C.c_size_t), ("q_heads", C.c_size_t), ("kv_heads", C.c_size_t),
        ("head_size", C.c_size_t), ("kv_strides", C.c_size_t * 4), ("scale", C.c_float),
    ]


def build():
    subprocess.run(["make", "-C", _HERE], check=True, stdout=subprocess.DEVNULL)


def load():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_SO):
        build()
    lib = C.CDLL(_SO)
    lib.oracle_dot_product_f32.restype = C.c_float
    lib.oracle_dot_product_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    lib.oracle_scalar_vector_mul_acc_f32.restype = None
    lib.oracle_scalar_vector_mul_acc_f32.argtypes = [C.c_float, C.c_void_p, C.c_float, C.c_void_p, C.c_size_t]
    lib.oracle_flash_attention_f32.restype = None
    lib.oracle_flash_attention_f32.argtypes = [C.c_void_p] * 4 + [C.c_float, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int, C.c_void_p]
    lib.oracle_assign.restype = C.c_int
    lib.oracle_assign.argtypes = [C.c_size_t] * 3 + [C.POINTER(C.c_size_t)] * 2
    lib.oracle_attention_run_bf16.restype = None
    lib.oracle_attention_run_bf16.argtypes = [C.POINTER(AttnDesc)] + [C.c_size_t] * 5
    lib.oracle_attention_run_threads_bf16.restype = None
    lib.oracle_attention_run_threads_bf16.argtypes = [C.POINTER(AttnDesc)] + [C.c_size_t] * 4
    lib.oracle_kv_append_bf16.restype = None
    lib.oracle_kv_append_bf16.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_size_t)] + [C.c_size_t] * 6 + [C.c_void_p]
    lib.oracle_merge_partials_f32.restype = None
    lib.oracle_merge_partials_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p]
    lib.oracle_rms_norm_f32.restype = None
    lib.oracle_rms_norm_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_float]
    lib.oracle_complex_mul_f32.restype = None
    lib.oracle_complex_mul_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
    lib.oracle_precompute_freqs_cis.restype = None
    lib.oracle_precompute_freqs_cis.argtypes = [C.c_size_t, C.c_size_t, C.c_float, C.c_void_p, C.c_int]
    lib.oracle_qk_norm_rope_append_bf16.restype = None
    lib.oracle_qk_norm_rope_append_bf16.argtypes = ([C.c_void_p] * 9 + [C.POINTER(C.c_size_t)] + [C.c_size_t] * 5
                                                     + [C.c_void_p, C.c_size_t, C.c_size_t, C.c_float])
    lib.oracle_matmul_nt_bf16.restype = None
    lib.oracle_matmul_nt_bf16.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p] + [C.c_size_t] * 5
    lib.oracle_f32_to_bf16.restype = C.c_uint16
    lib.oracle_f32_to_bf16.argtypes = [C.c_float]
    lib.oracle_f16_available.restype = C.c_int
    lib.oracle_f16_dot_product.restype = C.c_float
    lib.oracle_f16_dot_product.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    lib.oracle_f16_scalar_vector_mul_acc.restype = None
    lib.oracle_f16_scalar_vector_mul_acc.argtypes = [C.c_float, C.c_void_p, C.c_float, C.c_void_p]
    lib.oracle_f16_flash_attention.restype = None
    lib.oracle_f16_flash_attention.argtypes = [C.c_void_p] * 4 + [C.c_float, C.c_size_t, C.c_size_t, C.c_size_t]
    lib.oracle_f16_attention_run_threads.restype = C.c_double
    lib.oracle_f16_attention_run_threads.argtypes = (
        [C.c_void_p] * 5 + [C.c_size_t] * 3 + [C.POINTER(C.c_size_t), C.c_float] + [C.c_size_t] * 5)
    _lib = lib
    return lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def f32_to_bf16_bits(x):
    """float32 array -> uint16 bf16 bit patterns, round-to-nearest-even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def assign(length, num, idx):
    """compiler::assign::assign -> (begin, end) or None."""
    b, e = C.c_size_t(), C.c_size_t()
    ok = load().oracle_assign(length, num, idx, C.byref(b), C.byref(e))
    return (b.value, e.value) if ok else None


def flash_attention_f32(q, K, V, o, scale, position, stride=None, faithful_scale_defect=False):
    """One query row against keys 0..=position; updates `o` in place, returns LSE."""
    lib = load()
    length = q.shape[-1]
    stride = length if stride is None else stride
    lse = C.c_float()
    lib.oracle_flash_attention_f32(_ptr(q), _ptr(K), _ptr(V), _ptr(o), scale, length, stride,
                                   position, int(faithful_scale_defect), C.byref(lse))
    return lse.value


def attention_bf16(q, k, v, kv_strides, q_heads, kv_heads, scale, position_index,
                   position_interval, batch_size, max_batch=None, positions=None, threads=0,
                   serial_thread_ids=None):
    """The attention operator on uint16 bf16 buffers.

    q: [interval, max_batch, q_heads, D]; k, v: flat caches addressed by kv_strides
    (elements).  Returns (out bf16 bits like q, lse float32 [interval, max_batch, q_heads]).
    `serial_thread_ids=n` replays the reference's own test idiom instead of real
    threads: for tid in 0..n: run(.., n, tid).
    """
    lib = load()
    q = np.ascontiguousarray(q, dtype=np.uint16)
    interval, mb, hq, d = q.shape
    max_batch = mb if max_batch is None else max_batch
    out = np.zeros_like(q)
    lse = np.zeros((interval, mb, hq), dtype=np.float32)
    desc = AttnDesc()
    desc.q, desc.k, desc.v, desc.out, desc.lse = (_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse))
    pos_arr = None
    if positions is not None:
        pos_arr = np.ascontiguousarray(positions, dtype=np.int32)
    desc.positions = _ptr(pos_arr)
    desc.max_batch, desc.q_heads, desc.kv_heads, desc.head_size = max_batch, q_heads, kv_heads, d
    desc.kv_strides = (C.c_size_t * 4)(*kv_strides)
    desc.scale = scale
    if serial_thread_ids:
        for tid in range(serial_thread_ids):
            lib.oracle_attention_run_bf16(C.byref(desc), position_index, position_interval,
                                          batch_size, serial_thread_ids, tid)
    else:
        lib.oracle_attention_run_threads_bf16(C.byref(desc), position_index, position_interval,
                                              batch_size, threads)
    return out, lse


def kv_append_bf16(cache, src, kv_strides, max_batch, kv_heads, head_size, position_index,
                   position_interval, batch_size, positions=None):
    pos_arr = None if positions is None else np.ascontiguousarray(positions, dtype=np.int32)
    load().oracle_kv_append_bf16(_ptr(cache), _ptr(src), (C.c_size_t * 4)(*kv_strides), max_batch,
                                 kv_heads, head_size, position_index, position_interval,
                                 batch_size, _ptr(pos_arr))


def merge_partials(o_parts, lse_parts):
    """o_parts [P, rows, D] f32, lse_parts [P, rows] f32 -> (o [rows, D], lse [rows])."""
    o_parts = np.ascontiguousarray(o_parts, dtype=np.float32)
    lse_parts = np.ascontiguousarray(lse_parts, dtype=np.float32)
    p, rows, d = o_parts.shape
    o = np.zeros((rows, d), dtype=np.float32)
    lse = np.zeros((rows,), dtype=np.float32)
    load().oracle_merge_partials_f32(_ptr(o_parts), _ptr(lse_parts), p, rows, d, _ptr(o), _ptr(lse))
    return o, lse


def attention_f16_timed(q, k, v, kv_strides, q_heads, kv_heads, scale, position_index,
                        position_interval, batch_size, max_batch, positions=None, threads=0,
                        repeats=1):
    """AVX-512-FP16 kernel over IEEE-half uint16 buffers (64-byte aligned rows).

    Returns (out uint16 like q, seconds) or (None, -1.0) without avx512fp16.
    """
    lib = load()
    if not lib.oracle_f16_available():
        return None, -1.0
    out = aligned_empty(q.shape, np.uint16)
    pos_arr = None if positions is None else np.ascontiguousarray(positions, dtype=np.int32)
    secs = lib.oracle_f16_attention_run_threads(
        _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(pos_arr), max_batch, q_heads, kv_heads,
        (C.c_size_t * 4)(*kv_strides), scale, position_index, position_interval, batch_size,
        threads, repeats)
    return out, secs


def aligned_empty(shape, dtype, align=64):
    """numpy array whose data pointer is `align`-byte aligned (the reference's allocator
    aligns to 64 bytes, src/memory/allocator.rs:4-27, and the f16 kernel relies on it)."""
    dtype = np.dtype(dtype)
    n = int(np.prod(shape)) * dtype.itemsize
    raw = np.empty(n + align, dtype=np.uint8)
    off = (-raw.ctypes.data) % align
    return raw[off:off + n].view(dtype).reshape(shape)


def softmax_attention_f64(q, K, V, scale):
    """Independent two-pass float64 softmax attention of ONE query row over all rows
    of K/V; returns (o, lse).  Not derived from the reference: the cross-check."""
    s = (K.astype(np.float64) @ q.astype(np.float64)) * scale
    m = s.max()
    p = np.exp(s - m)
    d = p.sum()
    return (p / d) @ V.astype(np.float64), m + np.log(d)


def rope_table(dim, rows, theta, faithful_to_polar=False):
    """[rows, dim] float32 of interleaved (cos, sin) pairs (precompute_freqs_cis)."""
    out = np.zeros((rows, dim), dtype=np.float32)
    load().oracle_precompute_freqs_cis(dim, rows, theta, _ptr(out), int(faithful_to_polar))
    return out


def qk_norm_rope_append_bf16(q_in, k_in, v_in, k_cache, v_cache, rope, kv_strides, q_heads, kv_heads,
                             position_index, position_interval, batch_size, eps, q_weight=None,
                             k_weight=None, positions=None, max_batch=None):
    """RMSNorm + RoPE on the Q and K heads, K and V written into the caches (in place); returns q_out."""
    q_in = np.ascontiguousarray(q_in, dtype=np.uint16)
    interval, mb, hq, d = q_in.shape
    max_batch = mb if max_batch is None else max_batch
    q_out = np.zeros_like(q_in)
    pos = None if positions is None else np.ascontiguousarray(positions, dtype=np.int32)
    qw = None if q_weight is None else np.ascontiguousarray(q_weight, dtype=np.float32)
    kw = None if k_weight is None else np.ascontiguousarray(k_weight, dtype=np.float32)
    rope = np.ascontiguousarray(rope, dtype=np.float32)
    load().oracle_qk_norm_rope_append_bf16(
        _ptr(q_in), _ptr(np.ascontiguousarray(k_in, dtype=np.uint16)), _ptr(np.ascontiguousarray(v_in, dtype=np.uint16)),
        _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _ptr(qw), _ptr(kw), _ptr(rope), (C.c_size_t * 4)(*kv_strides),
        max_batch, q_heads, kv_heads, d, position_index, _ptr(pos), position_interval, batch_size, eps)
    return q_out


def matmul_nt_bf16(a, w_nt, residual=None, threads=None):
    """bf16 bits: (residual +) a[m, k] . w_nt[n, k]^T with fp32 accumulation, rounded once."""
    a = np.ascontiguousarray(a, dtype=np.uint16)
    w_nt = np.ascontiguousarray(w_nt, dtype=np.uint16)
    m, k = a.shape
    n = w_nt.shape[0]
    assert w_nt.shape[1] == k
    res = None if residual is None else np.ascontiguousarray(residual, dtype=np.uint16)
    out = np.zeros((m, n), dtype=np.uint16)
    threads = threads or min(os.cpu_count() or 1, 16)
    load().oracle_matmul_nt_bf16(_ptr(a), k, _ptr(w_nt), _ptr(res), n, _ptr(out), n, m, n, k, threads)
    return out
