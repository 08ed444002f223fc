"""The oracle's projection restatement (C = residual + A . W_nt^T, fp32 accumulation, one bf16
rounding) against float64 numpy, and the reference's own known-answer shapes for it (CPU only).

The reference's tests for these operators use all-ones operands: a row of k ones times a column
of k ones is k (src/compiler/mul/matmul_add.rs tests add a residual of ones: k + 1)."""
import numpy as np

import oracle


def _bits(a):
    return oracle.f32_to_bf16_bits(np.asarray(a, dtype=np.float32))


def test_all_ones_known_answers():
    for m, n, k in ((3, 32, 64), (6, 64, 128)):
        a, w = _bits(np.ones((m, k))), _bits(np.ones((n, k)))
        assert (oracle.bf16_bits_to_f32(oracle.matmul_nt_bf16(a, w)) == k).all()
        res = _bits(np.ones((m, n)))
        assert (oracle.bf16_bits_to_f32(oracle.matmul_nt_bf16(a, w, res)) == k + 1).all()


def test_against_float64_and_thread_split():
    rng = np.random.default_rng(5)
    a, w = _bits(rng.standard_normal((37, 192))), _bits(rng.standard_normal((50, 192)) * 0.1)
    res = _bits(rng.standard_normal((37, 50)))
    got1 = oracle.matmul_nt_bf16(a, w, res, threads=1)
    got5 = oracle.matmul_nt_bf16(a, w, res, threads=5)
    assert np.array_equal(got1, got5)   # the row split does not change a row's arithmetic
    ref = (oracle.bf16_bits_to_f32(a).astype(np.float64) @ oracle.bf16_bits_to_f32(w).astype(np.float64).T
           + oracle.bf16_bits_to_f32(res))
    g = oracle.bf16_bits_to_f32(got1)
    assert (np.abs(g - ref) <= np.abs(ref) * 2.0 ** -8 + 1e-5).all()   # half a bf16 step plus the fp32 sum's error
