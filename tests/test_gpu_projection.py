"""The tensor-core projections (MatMul3 with its fused norm + rope + cache write, MatMulAdd)
against the CPU oracle, through the C ABI (B200 only).

The oracle sums a dot product in k order in fp32; the tensor core sums the same fp32 products in
another order, so a result may land one bf16 step away from the oracle's.  For the fused
projection that step happens before the norm, so the bar is the one of the norm + rope kernel:
nearly all values bit-equal, the rest within a bf16 step of the larger member of their rotation
pair (the rotation mixes the pair, so a small output inherits the step of its large partner).
Rows and cache lines the kernels must not touch are bit-exact."""
import numpy as np
import pytest
import torch

import ellm_b200
import oracle
from ellm_b200.projection import MatMul3, MatMulAdd
from helpers import bits

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _close(got, want, exact_min, steps=1, atol=0.0):
    g32, w32 = oracle.bf16_bits_to_f32(got), oracle.bf16_bits_to_f32(want)
    assert np.isfinite(g32).all()
    exact = (got == want).mean()
    assert exact >= exact_min, exact
    assert (np.abs(g32 - w32) <= steps * np.abs(w32) * 2.0 ** -7 + atol).all(), np.abs(g32 - w32).max()


def _close_rotated(got, want):
    g32, w32 = oracle.bf16_bits_to_f32(got), oracle.bf16_bits_to_f32(want)
    assert np.isfinite(g32).all()
    assert (got == want).mean() >= 0.97, (got == want).mean()
    pair = np.abs(w32).reshape(-1, 2).max(axis=1, keepdims=True).repeat(2, axis=1).reshape(w32.shape)
    d = np.abs(g32 - w32)
    assert (d <= 2 * pair * 2.0 ** -7 + 1e-30).all(), d.max()
    assert d.mean() <= 2e-4, d.mean()


def _matmul_add(seed, interval, max_batch, batch, n, k, residual, in_place=False, a_pad=0, pairing=None):
    g = torch.Generator().manual_seed(seed)
    m = interval * max_batch
    a_full = torch.randn(m, k + a_pad, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16)
    res = torch.randn(m, n, generator=g).to(torch.bfloat16) if residual else None
    canary = torch.randn(m, n, generator=g).to(torch.bfloat16)
    want = oracle.matmul_nt_bf16(bits(a_full)[:, :k], bits(w), None if res is None else bits(res))
    da, dw = a_full.to(DEV), w.to(DEV)
    dres = None if res is None else res.to(DEV)
    out = dres if in_place else canary.to(DEV)
    op = MatMulAdd.new(da, dw, dres, out, m, n, k, max_batch=max_batch, a_row_stride=k + a_pad)
    if pairing is not None:
        op.set_pairing(pairing)
    op.run(0, interval, batch)
    got = bits(out).reshape(interval, max_batch, n)
    want = want.reshape(interval, max_batch, n)
    # the accumulated rounding of k fp32 additions, against values of size ~ sqrt(k) * 0.05
    _close(got[:, :batch], want[:, :batch], 0.99, atol=2e-5 * np.sqrt(k))
    if batch < max_batch:   # dead sequence slots keep what they held
        before = bits(res if in_place else canary).reshape(interval, max_batch, n)
        assert np.array_equal(got[:, batch:], before[:, batch:])
    assert op.kernel_stats()[0] == 1
    op.close()


def test_matmul_plain_ragged_edges():
    _matmul_add(1, interval=300, max_batch=1, batch=1, n=200, k=256, residual=False)


def test_matmul_add_residual_in_place_dead_slots():
    _matmul_add(2, interval=67, max_batch=3, batch=2, n=640, k=192, residual=True, in_place=True)


def test_matmul_add_strided_a_many_k_blocks():
    # 32 k-blocks go eight times round the 4-slot ring; 20 column tiles x 8 row tiles > SMs
    _matmul_add(3, interval=1024, max_batch=1, batch=1, n=5120, k=2048, residual=True, a_pad=64)


def test_matmul_decode_rows():
    # 64 k-blocks through a 48-slot ring, 128 CTAs of 16 columns
    _matmul_add(4, interval=1, max_batch=16, batch=16, n=2048, k=4096, residual=True)


def test_matmul_decode_one_row_odd_columns_in_place():
    _matmul_add(5, interval=1, max_batch=1, batch=1, n=200, k=128, residual=True, in_place=True)


def test_matmul_decode_dead_slots_no_residual():
    _matmul_add(6, interval=1, max_batch=5, batch=3, n=1024, k=512, residual=False)


@pytest.mark.parametrize("rows", [2, 8, 9])
def test_matmul_decode_row_counts_around_the_fragment_paths(rows):
    # up to 8 rows of a 16-column slice take the transposed products fed by 16-byte shared-memory loads,
    # 9 and more the ldmatrix loop
    _matmul_add(40 + rows, interval=1, max_batch=rows, batch=rows, n=1024, k=1024, residual=True)


def test_matmul_decode_long_rows_take_the_slice_in_two_passes():
    # 16 columns x 12288 do not fit shared memory at once: the slice comes in two passes over K
    _matmul_add(50, interval=1, max_batch=3, batch=3, n=256, k=12288, residual=True)


def _matmul3(seed, interval, max_batch, batch, q_heads, kv_heads, hidden, max_seq, position_index=0, positions=None,
             weights=True, one_matrix=False, pairing=None):
    g = torch.Generator().manual_seed(seed)
    m = interval * max_batch
    x = torch.randn(m, hidden, generator=g).to(torch.bfloat16)
    wq = (torch.randn(q_heads * 128, hidden, generator=g) * 0.05).to(torch.bfloat16)
    wk = (torch.randn(kv_heads * 128, hidden, generator=g) * 0.05).to(torch.bfloat16)
    wv = (torch.randn(kv_heads * 128, hidden, generator=g) * 0.05).to(torch.bfloat16)
    ck = torch.randn(max_batch, kv_heads, max_seq, 128, generator=g).to(torch.bfloat16)   # canaries
    cv = torch.randn(max_batch, kv_heads, max_seq, 128, generator=g).to(torch.bfloat16)
    qw = (1 + 0.02 * torch.randn(128, generator=g)).float() if weights else None
    kw = (1 + 0.02 * torch.randn(128, generator=g)).float() if weights else None
    rope = ellm_b200.precompute_freqs_cis(128, max_seq, 1e6)
    strides = [kv_heads * max_seq * 128, max_seq * 128, 128, 1]
    # oracle: the three projections, stored as bf16, then the norm + rope + cache-write step
    pq = oracle.matmul_nt_bf16(bits(x), bits(wq)).reshape(interval, max_batch, q_heads, 128)
    pk = oracle.matmul_nt_bf16(bits(x), bits(wk)).reshape(interval, max_batch, kv_heads, 128)
    pv = oracle.matmul_nt_bf16(bits(x), bits(wv)).reshape(interval, max_batch, kv_heads, 128)
    want_ck, want_cv = bits(ck).copy(), bits(cv).copy()
    want_q = oracle.qk_norm_rope_append_bf16(pq, pk, pv, want_ck, want_cv, rope, strides, q_heads, kv_heads,
                                             position_index, interval, batch, 1e-6,
                                             q_weight=None if qw is None else qw.numpy(),
                                             k_weight=None if kw is None else kw.numpy(), positions=positions,
                                             max_batch=max_batch)
    dx, dck, dcv = x.to(DEV), ck.to(DEV), cv.to(DEV)
    q_out = torch.zeros(interval, max_batch, q_heads, 128, dtype=torch.bfloat16, device=DEV)
    if one_matrix:   # Wq, Wk, Wv back to back in memory: a decode step streams them as one matrix
        wqkv = torch.cat([wq, wk, wv]).to(DEV)
        dwq, dwk, dwv = wqkv[:q_heads * 128], wqkv[q_heads * 128:(q_heads + kv_heads) * 128], wqkv[(q_heads + kv_heads) * 128:]
    else:
        dwq, dwk, dwv = wq.to(DEV), wk.to(DEV), wv.to(DEV)
    op = MatMul3.new(dx, dwq, q_out, dwk, dck, dwv, dcv, torch.from_numpy(rope).to(DEV), 128, m,
                     hidden, q_heads * 128, kv_heads * 128, kv_strides=strides, max_batch=max_batch, max_seq=max_seq,
                     rope_rows=max_seq, eps=1e-6, q_norm_weight=None if qw is None else qw.to(DEV),
                     k_norm_weight=None if kw is None else kw.to(DEV))
    if pairing is not None:
        op.set_pairing(pairing)
    if positions is None:
        op.run(position_index, interval, batch)
    else:
        op.run_ragged(torch.tensor(positions, dtype=torch.int32, device=DEV), interval, batch)
    # V: the projection itself, rounded once; rows of other positions / sequences bit-equal to the canaries
    _close(bits(dcv), want_cv, 0.99, atol=2e-5 * np.sqrt(hidden))
    touched_v = bits(dcv) != bits(cv)
    assert not touched_v[batch:].any()
    _close_rotated(bits(q_out)[:, :batch], want_q[:, :batch])
    _close_rotated(bits(dck), want_ck)
    assert (bits(q_out)[:, batch:] == 0).all()   # dead sequence slots untouched
    untouched = want_ck == bits(ck)              # cache rows the oracle left alone
    assert np.array_equal(bits(dck)[untouched], bits(ck)[untouched])
    op.close()


def test_matmul3_prefill_chunk():
    _matmul3(11, interval=200, max_batch=2, batch=2, q_heads=4, kv_heads=2, hidden=256, max_seq=256, position_index=37)


def test_matmul3_odd_head_counts_no_weights_dead_slot():
    _matmul3(12, interval=70, max_batch=3, batch=2, q_heads=3, kv_heads=1, hidden=128, max_seq=96, position_index=5,
             weights=False)


def test_matmul3_decode_ragged_positions():
    _matmul3(13, interval=1, max_batch=3, batch=3, q_heads=8, kv_heads=2, hidden=512, max_seq=300,
             positions=[0, 299, 128])


def test_matmul3_decode_model_shape_one_matrix():
    # 16 sequences, one dead; 5120 columns in slices of 48 over 107 CTAs; the ring wraps (32 k-blocks, 26 slots)
    _matmul3(15, interval=1, max_batch=16, batch=15, q_heads=32, kv_heads=4, hidden=2048, max_seq=64,
             positions=list(range(3, 48, 3)), one_matrix=True)


def test_matmul3_two_row_chunk_of_one_sequence():
    _matmul3(16, interval=2, max_batch=1, batch=1, q_heads=4, kv_heads=2, hidden=256, max_seq=40, position_index=17,
             one_matrix=True)


def test_matmul3_chunk_with_per_sequence_starts():
    # a prompt chunk of three sequences that start at different positions (tensor-memory kernel, both forms)
    for pairing in (0, 1):
        _matmul3(18, interval=60, max_batch=3, batch=3, q_heads=4, kv_heads=2, hidden=192, max_seq=128,
                 positions=[0, 17, 64], pairing=pairing)


def test_matmul3_model_shape():
    # the benchmark stack's layer shape on a short chunk: 40 heads of columns, 32 k-blocks
    _matmul3(14, interval=384, max_batch=1, batch=1, q_heads=32, kv_heads=4, hidden=2048, max_seq=512,
             position_index=100)


def test_cta_pairs_matmul_add():
    # two CTAs per 256 x 256 tile: ragged rows (300 = 256 + 44) and columns, then a many-tile case
    _matmul_add(21, interval=300, max_batch=1, batch=1, n=200, k=256, residual=False, pairing=1)
    _matmul_add(22, interval=67, max_batch=3, batch=2, n=640, k=192, residual=True, in_place=True, pairing=1)
    _matmul_add(23, interval=1024, max_batch=1, batch=1, n=5120, k=2048, residual=True, a_pad=64, pairing=1)


def test_cta_pairs_matmul3():
    _matmul3(24, interval=200, max_batch=2, batch=2, q_heads=4, kv_heads=2, hidden=256, max_seq=256, position_index=37, pairing=1)
    _matmul3(25, interval=70, max_batch=3, batch=2, q_heads=3, kv_heads=1, hidden=128, max_seq=96, position_index=5,
             weights=False, pairing=1)
    _matmul3(26, interval=384, max_batch=1, batch=1, q_heads=32, kv_heads=4, hidden=2048, max_seq=512, position_index=100,
             pairing=1)


def test_matmul_between_the_two_kernels_row_counts():
    # 17 .. 127 rows: more than the streaming kernel takes, less than one full tile of the other
    _matmul_add(7, interval=20, max_batch=2, batch=2, n=512, k=256, residual=True)
    _matmul3(17, interval=9, max_batch=3, batch=3, q_heads=4, kv_heads=2, hidden=256, max_seq=64, position_index=30)


def test_device_wait_timeout_is_reported_and_the_handle_stays_usable():
    """Failure detection without a fault: the loader leaves one operand block unloaded (a barrier that
    nothing signals), the wait on it runs out after the configured bound, every role leaves, tensor
    memory is released and the run reports ELLM_ERR_DEVICE_TIMEOUT.  The same handle then runs
    normally and matches the oracle."""
    from ellm_b200 import _lib as L
    g = torch.Generator().manual_seed(41)
    m, n, k = 256, 512, 256
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    op = MatMulAdd.new(a.to(DEV), w.to(DEV), None, out, m, n, k, max_batch=1)
    op.set_wait_timeout(200_000_000)   # 0.2 s
    op.debug_skip_load(2)
    with pytest.raises(ellm_b200.EllmError) as e:
        op.run(0, m, 1)
    assert e.value.status == L.ERR_DEVICE_TIMEOUT
    op.debug_skip_load(-1)
    op.run(0, m, 1)                    # same handle, same context
    _close(bits(out), oracle.matmul_nt_bf16(bits(a), bits(w)), 0.99, atol=2e-5 * np.sqrt(k))
    op.close()


def test_invalid_arguments():
    x = torch.zeros(128, 100, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(256, 100, dtype=torch.bfloat16, device=DEV)
    o = torch.zeros(128, 256, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ellm_b200.EllmError):   # k not a multiple of 64
        MatMulAdd.new(x, w, None, o, 128, 256, 100)
    x = torch.zeros(128, 128, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(256, 128, dtype=torch.bfloat16, device=DEV)
    op = MatMulAdd.new(x, w, None, o, 128, 256, 128, max_batch=4)
    with pytest.raises(ellm_b200.EllmError):   # more live sequences than slots
        op.run(0, 1, 5)
    with pytest.raises(ellm_b200.EllmError):   # more rows than the buffers hold
        op.run(0, 33, 4)
    op.run(0, 32, 4, cpu_num=8, thread_id=3)   # a worker that is not thread 0 launches nothing
    op.run(0, 0, 4)                            # an empty chunk and an empty batch are no work, not errors
    op.run(0, 1, 0)
    assert op.kernel_stats()[0] == 0
    op.close()


@pytest.mark.parametrize("interval,max_batch", [(1, 4), (1, 16), (160, 2)])
def test_matmul3_input_norm_equals_separate_norm(interval, max_batch):
    """The input norm inside the operator gives the bits of ellm_rms_norm followed by the operator."""
    g = torch.Generator().manual_seed(31)
    q_heads, kv_heads, hidden, max_seq = 8, 2, 1024, 256
    m = interval * max_batch
    x = (torch.randn(m, hidden, generator=g) * 3).to(torch.bfloat16).to(DEV)
    wqkv = (torch.randn((q_heads + 2 * kv_heads) * 128, hidden, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    wq, wk, wv = wqkv[:q_heads * 128], wqkv[q_heads * 128:(q_heads + kv_heads) * 128], wqkv[(q_heads + kv_heads) * 128:]
    rope = torch.from_numpy(ellm_b200.precompute_freqs_cis(128, max_seq, 1e6)).to(DEV)
    strides = [kv_heads * max_seq * 128, max_seq * 128, 128, 1]
    outs = []
    for fused in (False, True):
        ck = torch.zeros(max_batch, kv_heads, max_seq, 128, dtype=torch.bfloat16, device=DEV)
        cv = torch.zeros_like(ck)
        q_out = torch.zeros(interval, max_batch, q_heads, 128, dtype=torch.bfloat16, device=DEV)
        h = torch.zeros_like(x)
        if fused:
            op = MatMul3.new(x, wq, q_out, wk, ck, wv, cv, rope, 128, m, hidden, q_heads * 128, kv_heads * 128,
                             kv_strides=strides, max_batch=max_batch, max_seq=max_seq, rope_rows=max_seq,
                             input_norm_eps=1e-6, normed_scratch=h)
        else:
            ellm_b200.rms_norm(x, h, 1e-6)
            op = MatMul3.new(h, wq, q_out, wk, ck, wv, cv, rope, 128, m, hidden, q_heads * 128, kv_heads * 128,
                             kv_strides=strides, max_batch=max_batch, max_seq=max_seq, rope_rows=max_seq)
        op.run(7, interval, max_batch - 1 if max_batch > 2 else max_batch)
        outs.append((bits(q_out), bits(ck), bits(cv)))
        op.close()
    for a, b in zip(*outs):
        assert np.array_equal(a, b)
    assert outs[0][0].any() and outs[0][1].any()


@pytest.mark.parametrize("one_matrix", [True, False])
def test_matmul3_decode_fusion_equals_two_kernels(one_matrix):
    """A decode step finished inside the projection kernel (clusters of 8 CTAs per head) gives the bits
    of the projection kernel followed by the norm + rope + append kernel."""
    g = torch.Generator().manual_seed(51)
    q_heads, kv_heads, hidden, max_seq, batch = 8, 2, 1024, 128, 5
    x = torch.randn(batch, hidden, generator=g).to(torch.bfloat16).to(DEV)
    wqkv = (torch.randn((q_heads + 2 * kv_heads) * 128, hidden, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    wq, wk, wv = wqkv[:q_heads * 128], wqkv[q_heads * 128:(q_heads + kv_heads) * 128], wqkv[(q_heads + kv_heads) * 128:]
    if not one_matrix:
        wq, wk, wv = wq.clone(), wk.clone(), wv.clone()
    qw = (1 + 0.02 * torch.randn(128, generator=g)).float().to(DEV)
    kw = (1 + 0.02 * torch.randn(128, generator=g)).float().to(DEV)
    rope = torch.from_numpy(ellm_b200.precompute_freqs_cis(128, max_seq, 1e6)).to(DEV)
    strides = [kv_heads * max_seq * 128, max_seq * 128, 128, 1]
    positions = torch.tensor([0, 127, 64, 5, 99], dtype=torch.int32, device=DEV)
    outs = []
    for fused in (True, False):
        ck = torch.zeros(batch, kv_heads, max_seq, 128, dtype=torch.bfloat16, device=DEV)
        cv = torch.zeros_like(ck)
        q_out = torch.zeros(1, batch, q_heads, 128, dtype=torch.bfloat16, device=DEV)
        op = MatMul3.new(x, wq, q_out, wk, ck, wv, cv, rope, 128, batch, hidden, q_heads * 128, kv_heads * 128,
                         kv_strides=strides, max_batch=batch, max_seq=max_seq, rope_rows=max_seq, q_norm_weight=qw,
                         k_norm_weight=kw, input_norm_eps=1e-6, normed_scratch=torch.zeros_like(x))
        op.set_decode_fusion(fused)
        op.run_ragged(positions, 1, batch - 1)
        outs.append((bits(q_out), bits(ck), bits(cv), op.kernel_stats()[0]))
        op.close()
    for a, b in zip(outs[0][:3], outs[1][:3]):
        assert np.array_equal(a, b)
    assert outs[0][0][0, :batch - 1].any() and not outs[0][0][0, batch - 1:].any()   # the dead slot stays untouched
    assert outs[0][3] == (1 if one_matrix else 3)


def test_smallest_k_and_plain_state_buffers():
    """One 64-wide k-block; and K / V landing in plain [rows x Nkv] state buffers like the reference's
    k_state / v_state: the cache strides [Nkv, 128, max_batch * Nkv, 1] with position_index 0 express that."""
    _matmul_add(61, interval=200, max_batch=1, batch=1, n=384, k=64, residual=True)
    _matmul_add(62, interval=1, max_batch=3, batch=3, n=384, k=64, residual=True)
    g = torch.Generator().manual_seed(63)
    interval, mb, hq, hkv, hidden = 40, 2, 4, 2, 128
    m, nkv = interval * mb, hkv * 128
    x = torch.randn(m, hidden, generator=g).to(torch.bfloat16)
    wq = (torch.randn(hq * 128, hidden, generator=g) * 0.05).to(torch.bfloat16)
    wk = (torch.randn(nkv, hidden, generator=g) * 0.05).to(torch.bfloat16)
    wv = (torch.randn(nkv, hidden, generator=g) * 0.05).to(torch.bfloat16)
    rope = ellm_b200.precompute_freqs_cis(128, interval, 1e6)
    k_state = torch.zeros(m, nkv, dtype=torch.bfloat16, device=DEV)
    v_state = torch.zeros_like(k_state)
    q = torch.zeros(interval, mb, hq, 128, dtype=torch.bfloat16, device=DEV)
    op = MatMul3.new(x.to(DEV), wq.to(DEV), q, wk.to(DEV), k_state, wv.to(DEV), v_state, torch.from_numpy(rope).to(DEV), 128, m,
                     hidden, hq * 128, nkv, kv_strides=[nkv, 128, mb * nkv, 1], max_batch=mb, max_seq=interval,
                     rope_rows=interval)
    op.run(0, interval, mb)
    want_v = oracle.matmul_nt_bf16(bits(x), bits(wv))
    _close(bits(v_state), want_v, 0.99, atol=2e-5 * np.sqrt(hidden))
    # K rows: norm + rotation of the projected rows, row m = (chunk row r, sequence b) rotated at position r
    pk = oracle.matmul_nt_bf16(bits(x), bits(wk)).reshape(interval, mb, hkv, 128)
    pq = oracle.matmul_nt_bf16(bits(x), bits(wq)).reshape(interval, mb, hq, 128)
    ck = np.zeros((m, nkv), np.uint16)
    cv = np.zeros((m, nkv), np.uint16)
    oracle.qk_norm_rope_append_bf16(pq, pk, want_v.reshape(interval, mb, hkv, 128), ck, cv, rope, [nkv, 128, mb * nkv, 1], hq, hkv,
                                    0, interval, mb, 1e-6, max_batch=mb)
    assert np.array_equal(cv, want_v)
    _close_rotated(bits(k_state), ck)
    op.close()
