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

    def set_pairing(self, mode):
        """CTA pairs per 256 x 256 tile in the tensor-memory kernel: -1 auto, 0 never, 1 whenever possible."""
        L.check(self._lib.ellm_matmul_set_pairing(self._h, self._which, int(mode)))

    def debug_skip_load(self, item):
        L.check(self._lib.ellm_matmul_debug_skip_load(self._h, self._which, int(item)))

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

    def set_decode_fusion(self, on):
        """Decode steps: head norm + rope + cache write inside the projection kernel (default) or as a second kernel."""
        L.check(self._lib.ellm_matmul3_set_decode_fusion(self._h, 1 if on else 0))

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


def main():
    """Times the two projection operators at one layer's shape (defaults: BASELINE configs[3]):

        python -m ellm_b200.projection --rows 32768        # tcgen05 kernel, a prefill chunk
        python -m ellm_b200.projection --rows 1            # weight-streaming kernel, a decode step
    """
    import argparse
    import json

    import torch

    from .rope import precompute_freqs_cis
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--q-heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--weight-sets", type=int, default=8, help="rotated so that decode steps stream weights from HBM, not L2")
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    S, hidden, qd, kd = args.rows, args.hidden, args.q_heads * 128, args.kv_heads * 128
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(S, hidden, device=dev, generator=g).to(torch.bfloat16)
    a = torch.randn(S, qd, device=dev, generator=g).to(torch.bfloat16)
    y = torch.zeros(S, hidden, dtype=torch.bfloat16, device=dev)
    q = torch.zeros(S, 1, args.q_heads, 128, dtype=torch.bfloat16, device=dev)
    max_seq = max(S, 64)
    ck = torch.zeros(1, args.kv_heads, max_seq, 128, dtype=torch.bfloat16, device=dev)
    cv = torch.zeros_like(ck)
    strides = [args.kv_heads * max_seq * 128, max_seq * 128, 128, 1]
    rope = torch.from_numpy(precompute_freqs_cis(128, max_seq, 1e6)).to(dev)
    ones = torch.ones(128, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    sets = args.weight_sets if S <= 16 else 1
    qkv_ops, out_ops = [], []
    for _ in range(sets):
        w = (torch.randn(qd + 2 * kd, hidden, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        wo = (torch.randn(hidden, qd, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        qkv_ops.append(MatMul3.new(x, w[:qd], q, w[qd:qd + kd], ck, w[qd + kd:], cv, rope, 128, S, hidden, qd, kd,
                                   kv_strides=strides, max_batch=1, max_seq=max_seq, rope_rows=max_seq, q_norm_weight=ones,
                                   k_norm_weight=ones, stream=stream, async_=True))
        out_ops.append(MatMulAdd.new(a, wo, y, y, S, hidden, qd, max_batch=1, stream=stream, async_=True))

    def timed(ops):
        for op in ops:
            op.run(0, S, 1)
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.reps):
            for op in ops:
                op.run(0, S, 1)
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / (args.reps * len(ops))

    t3, ta = timed(qkv_ops), timed(out_ops)
    for op in qkv_ops + out_ops:
        op.check()
    print(json.dumps({
        "rows": S, "hidden": hidden, "q_heads": args.q_heads, "kv_heads": args.kv_heads,
        "matmul3_ms": t3, "matmul3_tflops": 2.0 * S * hidden * (qd + 2 * kd) / t3 / 1e9,
        "matmul3_weight_gbs": (qd + 2 * kd) * hidden * 2 / t3 / 1e6,
        "matmul_add_ms": ta, "matmul_add_tflops": 2.0 * S * hidden * qd / ta / 1e9,
        "matmul_add_weight_gbs": hidden * qd * 2 / ta / 1e6}))
    for op in qkv_ops + out_ops:
        op.close()


if __name__ == "__main__":
    main()
