"""Host-side mirror of the reference's attention operator over the C ABI.

`Attention.new(...)` takes the arguments of the reference's `Attention::new`
(src/compiler/mul/attention.rs:41-67) in the same order and with the same
meaning, and `run(position_index, position_interval, batch_size, cpu_num,
thread_id)` is its `run` (attention.rs:69-76).  What a device needs beyond that
(cache capacity, the new K/V rows to append, an LSE output, a stream) are keyword
arguments.  Tensors are torch CUDA tensors used purely as device buffers; raw
integer device pointers work too.
"""
import ctypes as C

from . import _lib as L


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return x.data_ptr()


class Attention:
    def __init__(self):
        raise TypeError("use Attention.new(...)")

    @classmethod
    def new(cls, q_ptr, k_ptr, v_ptr, output_ptr, batch_size, attention_head_num, kv_head_num,
            head_size, kv_strides, inverse_sqrt_head, *, max_seq, max_interval=1, lse=None,
            k_new=None, v_new=None, device=0, stream=None, async_=False,
            prefill_kernel=L.PREFILL_AUTO, early_stream=False):
        self = object.__new__(cls)
        lib = L.load()
        d = L.AttnDesc()
        d.q, d.k_cache, d.v_cache, d.out = _ptr(q_ptr), _ptr(k_ptr), _ptr(v_ptr), _ptr(output_ptr)
        d.lse, d.k_new, d.v_new = _ptr(lse), _ptr(k_new), _ptr(v_new)
        d.max_batch, d.q_heads, d.kv_heads, d.head_size = batch_size, attention_head_num, kv_head_num, head_size
        d.kv_strides = (C.c_size_t * 4)(*[int(s) for s in kv_strides])
        d.max_seq, d.max_interval = max_seq, max_interval
        d.scale = float(inverse_sqrt_head)
        d.dtype, d.device = L.DTYPE_BF16, device
        d.stream = stream
        d.async_ = 1 if async_ else 0
        d.prefill_kernel = prefill_kernel
        handle = C.c_void_p()
        L.check(lib.ellm_attn_create(C.byref(d), C.byref(handle)))
        self._lib, self._h, self.desc = lib, handle, d
        if early_stream:   # see "decode_early_stream" in ellm_attn.h: the caller vouches for what precedes a decode step
            L.check(lib.ellm_attn_set_option(handle, b"decode_early_stream", 1))
        # keep the buffers alive as long as the operator (the reference leaks them instead)
        self._keep = (q_ptr, k_ptr, v_ptr, output_ptr, lse, k_new, v_new)
        return self

    def run(self, position_index, position_interval, batch_size, cpu_num=1, thread_id=0):
        L.check(self._lib.ellm_attn_run(self._h, position_index, position_interval, batch_size,
                                        cpu_num, thread_id))

    def run_ragged(self, positions, position_interval, batch_size, cpu_num=1, thread_id=0):
        L.check(self._lib.ellm_attn_run_ragged(self._h, _ptr(positions), position_interval,
                                               batch_size, cpu_num, thread_id))

    def run_window(self, position_index, position_interval, batch_size, key_begin, key_end,
                   o_part, lse_part):
        L.check(self._lib.ellm_attn_run_window(self._h, position_index, position_interval,
                                               batch_size, key_begin, key_end, _ptr(o_part),
                                               _ptr(lse_part)))

    def run_window_q(self, q, position_index, position_interval, batch_size, key_begin, key_end,
                     o_part, lse_part):
        """run_window with the queries read from `q` (same shape as the bound q buffer)."""
        L.check(self._lib.ellm_attn_run_window_q(self._h, _ptr(q), position_index, position_interval,
                                                 batch_size, key_begin, key_end, _ptr(o_part),
                                                 _ptr(lse_part)))

    def check(self):
        """Waits for the handle's stream; raises EllmError(ERR_DEVICE_TIMEOUT) if a bounded
        device-side wait of a kernel enqueued since the last check ran out (async handles)."""
        L.check(self._lib.ellm_attn_check(self._h))

    def run_host(self, q_host, out_host, position_index, position_interval, batch_size, *,
                 k_new_host=None, v_new_host=None, lse_host=None, positions_host=None):
        L.check(self._lib.ellm_attn_run_host(self._h, _ptr(q_host), _ptr(k_new_host),
                                             _ptr(v_new_host), _ptr(out_host), _ptr(lse_host),
                                             _ptr(positions_host), position_index,
                                             position_interval, batch_size))

    def bind_host(self, q_host, out_host, position_index, position_interval, batch_size, *,
                  k_new_host=None, v_new_host=None, lse_host=None, positions_host=None):
        """run_host for a loop that reuses the same host buffers: the arguments are converted once and the
        returned callable makes the one C call per step (a decode loop rewrites the buffers' contents, not
        the buffers).  The buffers are kept alive by the callable."""
        fn, h = self._lib.ellm_attn_run_host, self._h
        args = (C.c_void_p(_ptr(q_host)), C.c_void_p(_ptr(k_new_host)), C.c_void_p(_ptr(v_new_host)),
                C.c_void_p(_ptr(out_host)), C.c_void_p(_ptr(lse_host)), C.c_void_p(_ptr(positions_host)),
                C.c_size_t(position_index), C.c_size_t(position_interval), C.c_size_t(batch_size))
        keep = (q_host, k_new_host, v_new_host, out_host, lse_host, positions_host)

        def step(_keep=keep):
            status = fn(h, *args)
            if status:
                L.check(status)
        return step

    def set_option(self, name, value):
        L.check(self._lib.ellm_attn_set_option(self._h, name.encode(), int(value)))

    def set_profiling(self, on):
        L.check(self._lib.ellm_attn_set_profiling(self._h, 1 if on else 0))

    def kernel_stats(self):
        """{kernel name: (launches, timed launches, total ms of the timed ones)}"""
        out = {}
        for i, name in enumerate(L.KERNEL_NAMES):
            n, t, ms = C.c_uint64(), C.c_uint64(), C.c_double()
            L.check(self._lib.ellm_attn_kernel_stats(self._h, i, C.byref(n), C.byref(t), C.byref(ms)))
            out[name] = (n.value, t.value, ms.value)
        return out

    def close(self):
        if self._h:
            self._lib.ellm_attn_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def kv_append(cache, src, kv_strides, max_batch, kv_heads, head_size, max_seq, position_index,
              position_interval, batch_size, positions=None, device=0, stream=None):
    lib = L.load()
    L.check(lib.ellm_kv_append(_ptr(cache), _ptr(src), (C.c_size_t * 4)(*[int(s) for s in kv_strides]),
                               max_batch, kv_heads, head_size, max_seq, position_index,
                               _ptr(positions), position_interval, batch_size, device, stream))


def merge_partials(o_parts, lse_parts, out, lse_out=None, device=0, stream=None, out_f32=False):
    """o_parts [parts, rows, 128] fp32, lse_parts [parts, rows] fp32 -> out [rows, 128] bf16
    (or fp32 with out_f32=True)."""
    parts, rows, d = o_parts.shape
    fn = L.load().ellm_attn_merge_partials_f32 if out_f32 else L.load().ellm_attn_merge_partials
    L.check(fn(_ptr(o_parts), _ptr(lse_parts), parts, rows, d, _ptr(out), _ptr(lse_out), device, stream))


def merge_partials_list(o_parts, lse_parts, out, lse_out=None, device=0, stream=None, out_f32=False):
    """Combine of parts held in separate buffers: o_parts a list of [rows, 128] fp32 tensors,
    lse_parts the matching [rows] fp32 tensors (at most 16); out [rows, 128] bf16 or fp32."""
    n = len(o_parts)
    rows = o_parts[0].numel() // 128
    po = (C.c_void_p * n)(*[_ptr(t) for t in o_parts])
    pl = (C.c_void_p * n)(*[_ptr(t) for t in lse_parts])
    L.check(L.load().ellm_attn_merge_partials_list(po, pl, n, rows, 128, _ptr(out), 1 if out_f32 else 0,
                                                   _ptr(lse_out), device, stream))


def decode_noalloc(q, k_cache, v_cache, out, batch_size, q_heads, kv_heads, head_size, kv_strides,
                   scale, *, max_seq, positions=None, position_index=0, lse=None, device=0,
                   stream=None):
    """One decode step without any device allocation (ellm_attn_decode_noalloc).

    For callers that may not allocate at run time - a serving loop whose memory was all
    planned and handed out up front, or a process in which another allocator already owns
    the GPU's memory.  The split-KV partials go to a fixed array inside the library, shared
    by every call on the device, so calls must not overlap on the GPU; sizes beyond the
    array (see NOALLOC_MAX_SLOTS / NOALLOC_MAX_BATCH) raise EllmError(ERR_UNSUPPORTED).
    The new token's K/V must already be in the cache.  Only enqueues; no synchronise.
    """
    L.check(L.load().ellm_attn_decode_noalloc(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(lse), _ptr(positions), position_index,
        batch_size, q_heads, kv_heads, head_size, (C.c_size_t * 4)(*[int(s) for s in kv_strides]),
        max_seq, float(scale), device, stream))


def qk_norm_rope_append(q_in, k_in, v_in, q_out, k_cache, v_cache, rope, kv_strides, max_batch, q_heads,
                        kv_heads, head_size, max_seq, position_index, position_interval, batch_size, eps, *,
                        q_weight=None, k_weight=None, positions=None, q_in_row_stride=0, kv_in_row_stride=0,
                        device=0, stream=None):
    """Per-head RMSNorm + interleaved RoPE on Q and K, K and V written into the cache
    (ellm_qk_norm_rope_append); rope is the fp32 [rows, 128] table of rope.precompute_freqs_cis."""
    L.check(L.load().ellm_qk_norm_rope_append(
        _ptr(q_in), _ptr(k_in), _ptr(v_in), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _ptr(q_weight),
        _ptr(k_weight), _ptr(rope), rope.shape[0], (C.c_size_t * 4)(*[int(s) for s in kv_strides]), max_batch,
        q_heads, kv_heads, head_size, max_seq, position_index, _ptr(positions), position_interval,
        batch_size, float(eps), q_in_row_stride, kv_in_row_stride, device, stream))


def rms_norm(x, y, eps, device=0, stream=None):
    """y = x / (sqrt(mean x^2) + eps) per row of a [rows, length] bf16 matrix (ellm_rms_norm)."""
    rows, length = x.shape
    L.check(L.load().ellm_rms_norm(_ptr(x), _ptr(y), rows, length, float(eps), device, stream))
