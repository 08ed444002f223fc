"""Host-side mirror of the reference's projection operators over the C ABI of include/ellm_proj.h.

`MatMul3.new(...)` follows the reference's `MatMul3::new` (src/compiler/mul/matmul3.rs:60-119):
hidden, the three N x K weights and the Q output first, then the rope table and the shapes
(head_dim, m_row, col, b_q_row, b_kv_row); K and V go into the static cache instead of separate
state buffers.  `MatMulAdd.new(...)` follows `MatMulAdd::new` (src/compiler/mul/matmul_add.rs:60-126):
A, W_nt, residual, output, then m_max, n_max, k_max.  Both have the `run(position_index,
position_interval, batch_size, cpu_num, thread_id)` of every reference operator.  Tensors are
torch CUDA tensors used as device buffers; raw integer device pointers work too.
"""
import ctypes as C

from . import _lib as L
from .attention import _ptr


class _Projection:
    _which = 0
    _destroy = None

    def __init__(self):
        raise TypeError("use .new(...)")

    def set_profiling(self, on):
        L.check(self._lib.ellm_matmul_set_profiling(self._h, self._which, 1 if on else 0))

    def kernel_stats(self):
        """(launches, timed launches, device milliseconds of the timed ones)."""
        n, t, ms = C.c_uint64(), C.c_uint64(), C.c_double()
        L.check(self._lib.ellm_matmul_kernel_stats(self._h, self._which, C.byref(n), C.byref(t), C.byref(ms)))
        return n.value, t.value, ms.value

    def check(self):
        """Waits for the stream; raises if a device-side wait ran out since the last check."""
        L.check(self._lib.ellm_matmul_check(self._h, self._which))

    def set_wait_timeout(self, ns):
        L.check(self._lib.ellm_matmul_set_wait_timeout(self._h, self._which, int(ns)))

    def close(self):
        if self._h:
            getattr(self._lib, self._destroy)(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class MatMul3(_Projection):
    _which = 0
    _destroy = "ellm_matmul3_destroy"

    @classmethod
    def new(cls, hidden_ptr, q_weight_ptr_nt, q_state_ptr, k_weight_ptr_nt, k_cache, v_weight_ptr_nt, v_cache,
            rope_ptr, head_dim, m_row, col, b_q_row, b_kv_row, *, kv_strides, max_batch, max_seq, rope_rows,
            eps=1e-6, q_norm_weight=None, k_norm_weight=None, hidden_row_stride=0, device=0, stream=None,
            async_=False, input_norm_eps=None, normed_scratch=None):
        """input_norm_eps: when given, hidden_ptr is the layer's un-normalised input and the operator
        applies the weight-free RMS norm itself (normed_scratch [m_row, col] is then required)."""
        self = object.__new__(cls)
        lib = L.load()
        d = L.MatMul3Desc()
        d.hidden, d.hidden_row_stride = _ptr(hidden_ptr), hidden_row_stride
        d.wq_nt, d.wk_nt, d.wv_nt = _ptr(q_weight_ptr_nt), _ptr(k_weight_ptr_nt), _ptr(v_weight_ptr_nt)
        d.q_state, d.k_cache, d.v_cache = _ptr(q_state_ptr), _ptr(k_cache), _ptr(v_cache)
        d.kv_strides = (C.c_size_t * 4)(*[int(s) for s in kv_strides])
        d.rope, d.rope_rows = _ptr(rope_ptr), rope_rows
        d.q_norm_weight, d.k_norm_weight = _ptr(q_norm_weight), _ptr(k_norm_weight)
        d.head_dim, d.m_row, d.col, d.b_q_row, d.b_kv_row = head_dim, m_row, col, b_q_row, b_kv_row
        d.max_batch, d.max_seq, d.eps = max_batch, max_seq, float(eps)
        d.device, d.stream, d.async_ = device, stream, 1 if async_ else 0
        if input_norm_eps is not None:
            d.input_norm, d.input_norm_eps, d.normed_scratch = 1, float(input_norm_eps), _ptr(normed_scratch)
        handle = C.c_void_p()
        L.check(lib.ellm_matmul3_create(C.byref(d), C.byref(handle)))
        self._lib, self._h, self.desc = lib, handle, d
        self._keep = (hidden_ptr, q_weight_ptr_nt, q_state_ptr, k_weight_ptr_nt, k_cache, v_weight_ptr_nt, v_cache,
                      rope_ptr, q_norm_weight, k_norm_weight, normed_scratch)
        return self

    def run(self, position_index, position_interval, batch_size, cpu_num=1, thread_id=0):
        L.check(self._lib.ellm_matmul3_run(self._h, position_index, position_interval, batch_size, cpu_num, thread_id))

    def run_ragged(self, positions, position_interval, batch_size, cpu_num=1, thread_id=0):
        L.check(self._lib.ellm_matmul3_run_ragged(self._h, _ptr(positions), position_interval, batch_size, cpu_num,
                                                  thread_id))


class MatMulAdd(_Projection):
    _which = 1
    _destroy = "ellm_matmul_add_destroy"

    @classmethod
    def new(cls, ptr1, ptr2_nt, ptr3, output_ptr, m_max, n_max, k_max, *, max_batch=None, a_row_stride=0,
            residual_row_stride=0, output_row_stride=0, device=0, stream=None, async_=False):
        """output = ptr3 (residual, may be None) + ptr1 [m, k] . ptr2_nt [n, k]^T."""
        self = object.__new__(cls)
        lib = L.load()
        d = L.MatMulAddDesc()
        d.a, d.a_row_stride, d.w_nt = _ptr(ptr1), a_row_stride, _ptr(ptr2_nt)
        d.residual, d.residual_row_stride = _ptr(ptr3), residual_row_stride
        d.output, d.output_row_stride = _ptr(output_ptr), output_row_stride
        d.m_max, d.n_max, d.k_max = m_max, n_max, k_max
        d.max_batch = m_max if max_batch is None else max_batch
        d.device, d.stream, d.async_ = device, stream, 1 if async_ else 0
        handle = C.c_void_p()
        L.check(lib.ellm_matmul_add_create(C.byref(d), C.byref(handle)))
        self._lib, self._h, self.desc = lib, handle, d
        self._keep = (ptr1, ptr2_nt, ptr3, output_ptr)
        return self

    def run(self, position_index, position_interval, batch_size, cpu_num=1, thread_id=0):
        L.check(self._lib.ellm_matmul_add_run(self._h, position_index, position_interval, batch_size, cpu_num,
                                              thread_id))
