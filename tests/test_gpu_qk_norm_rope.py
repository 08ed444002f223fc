"""The fused RMSNorm + RoPE + cache-write kernel against the CPU oracle (B200 only).

The kernel sums the squares with a warp butterfly, the oracle sequentially, so a normalised
value may land one bf16 step away; V rows and everything the kernel must not touch are
bit-exact."""
import numpy as np
import pytest
import torch

import ellm_b200
import oracle
from helpers import bits, from_bits

pytestmark = pytest.mark.gpu


def _case(seed, S, B, max_batch, Hq, Hkv, max_seq, position_index=0, positions=None, weights=True):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(S, max_batch, Hq, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(S, max_batch, Hkv, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(S, max_batch, Hkv, 128, generator=g).to(torch.bfloat16)
    ck = torch.randn(max_batch, Hkv, max_seq, 128, generator=g).to(torch.bfloat16)   # canaries
    cv = torch.randn(max_batch, Hkv, max_seq, 128, generator=g).to(torch.bfloat16)
    qw = (1 + 0.02 * torch.randn(128, generator=g)).float() if weights else None
    kw = (1 + 0.02 * torch.randn(128, generator=g)).float() if weights else None
    rope = ellm_b200.precompute_freqs_cis(128, max_seq, 1e6)
    strides = [Hkv * max_seq * 128, max_seq * 128, 128, 1]
    want_ck, want_cv = bits(ck).copy(), bits(cv).copy()
    want_q = oracle.qk_norm_rope_append_bf16(bits(q), bits(k), bits(v), want_ck, want_cv, rope, strides, Hq, Hkv,
                                             position_index, S, B, 1e-6, q_weight=None if qw is None else qw.numpy(),
                                             k_weight=None if kw is None else kw.numpy(), positions=positions, max_batch=max_batch)
    dev = torch.device("cuda:0")
    dq, dck, dcv = q.to(dev), ck.to(dev), cv.to(dev)
    q_out = torch.zeros_like(dq)
    pos = None if positions is None else torch.tensor(positions, dtype=torch.int32, device=dev)
    ellm_b200.qk_norm_rope_append(dq, k.to(dev), v.to(dev), q_out, dck, dcv, torch.from_numpy(rope).to(dev), strides,
                                  max_batch, Hq, Hkv, 128, max_seq, position_index, S, B, 1e-6,
                                  q_weight=None if qw is None else qw.to(dev), k_weight=None if kw is None else kw.to(dev),
                                  positions=pos)
    torch.cuda.synchronize()
    assert np.array_equal(bits(dcv), want_cv), "V rows / untouched rows differ"
    for got, want in ((bits(q_out)[:, :B], want_q[:, :B]), (bits(dck), want_ck)):
        g32, w32 = oracle.bf16_bits_to_f32(got), oracle.bf16_bits_to_f32(want)
        assert np.isfinite(g32).all()
        exact = (got == want).mean()
        assert exact >= 0.98, exact
        assert (np.abs(g32 - w32) <= np.abs(w32) * 2.0 ** -7 + 1e-30).all()   # at most one bf16 step
    assert (bits(q_out)[:, B:] == 0).all()   # dead batch slots untouched


@pytest.mark.parametrize("weights", [True, False])
def test_prefill_chunk(weights):
    _case(1, S=37, B=2, max_batch=3, Hq=8, Hkv=2, max_seq=64, position_index=9, weights=weights)


def test_decode_ragged_positions():
    _case(2, S=1, B=3, max_batch=3, Hq=32, Hkv=4, max_seq=300, positions=[0, 299, 128])


def test_feeds_attention_end_to_end():
    """norm+rope+append then attention == the oracle's two steps chained."""
    dev = torch.device("cuda:0")
    S, B, Hq, Hkv, max_seq = 150, 1, 8, 2, 160
    g = torch.Generator().manual_seed(5)
    q = torch.randn(S, B, Hq, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(S, B, Hkv, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(S, B, Hkv, 128, generator=g).to(torch.bfloat16)
    rope = ellm_b200.precompute_freqs_cis(128, max_seq, 1e6)
    strides = [Hkv * max_seq * 128, max_seq * 128, 128, 1]
    ck = np.zeros((B, Hkv, max_seq, 128), np.uint16); cv = np.zeros_like(ck)
    want_q = oracle.qk_norm_rope_append_bf16(bits(q), bits(k), bits(v), ck, cv, rope, strides, Hq, Hkv, 0, S, B, 1e-6)
    scale = 1 / np.sqrt(128.0)
    want_o, want_l = oracle.attention_bf16(want_q, ck, cv, strides, Hq, Hkv, scale, 0, S, B)
    dq = q.to(dev); dck = torch.zeros(B, Hkv, max_seq, 128, dtype=torch.bfloat16, device=dev); dcv = torch.zeros_like(dck)
    out = torch.zeros_like(dq); lse = torch.zeros(S, B, Hq, dtype=torch.float32, device=dev)
    ellm_b200.qk_norm_rope_append(dq, k.to(dev), v.to(dev), dq, dck, dcv, torch.from_numpy(rope).to(dev), strides, B, Hq, Hkv,
                                  128, max_seq, 0, S, B, 1e-6)   # in place on q
    op = ellm_b200.Attention.new(dq, dck, dcv, out, B, Hq, Hkv, 128, strides, scale, max_seq=max_seq, max_interval=S, lse=lse)
    op.run(0, S, B, 1, 0)
    d = np.abs(out.float().cpu().numpy() - oracle.bf16_bits_to_f32(want_o))
    assert d.max() <= 2e-2 and d.mean() <= 2e-3
    assert np.abs(lse.cpu().numpy() - want_l).max() <= 2e-2   # one-bf16-step differences in normalised Q/K move the scores


def test_rms_norm_rows_against_oracle():
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(9)
    for rows, length in ((1, 8), (5, 2048), (37, 4096), (3, 264)):
        x = (torch.randn(rows, length, generator=g) * 3).to(torch.bfloat16)
        xf = x.float().numpy()
        want = np.empty_like(xf)
        for r in range(rows):
            oracle.load().oracle_rms_norm_f32(xf[r].ctypes.data, want[r].ctypes.data, length, 1e-6)
        want_bits = oracle.f32_to_bf16_bits(want)
        y = torch.zeros(rows, length, dtype=torch.bfloat16, device=dev)
        ellm_b200.rms_norm(x.to(dev), y, 1e-6)
        torch.cuda.synchronize()
        got = bits(y)
        assert (got == want_bits).mean() >= 0.98
        g32, w32 = oracle.bf16_bits_to_f32(got), oracle.bf16_bits_to_f32(want_bits)
        assert (np.abs(g32 - w32) <= np.abs(w32) * 2.0 ** -7 + 1e-30).all()


def test_inputs_as_column_blocks_of_one_projection_output():
    """q, k, v given as column blocks of a fused [rows, (Hq + 2 Hkv) * 128] matrix equal the contiguous form."""
    dev = torch.device("cuda:0")
    S, B, Hq, Hkv, max_seq = 9, 2, 4, 2, 16
    g = torch.Generator().manual_seed(10)
    qkv = torch.randn(S * B, (Hq + 2 * Hkv) * 128, generator=g).to(torch.bfloat16).to(dev)
    qd, kd = Hq * 128, Hkv * 128
    rope = torch.from_numpy(ellm_b200.precompute_freqs_cis(128, max_seq, 1e6)).to(dev)
    strides = [Hkv * max_seq * 128, max_seq * 128, 128, 1]
    outs = []
    for fused in (False, True):
        ck = torch.zeros(B, Hkv, max_seq, 128, dtype=torch.bfloat16, device=dev); cv = torch.zeros_like(ck)
        q_out = torch.zeros(S, B, Hq, 128, dtype=torch.bfloat16, device=dev)
        if fused:
            ellm_b200.qk_norm_rope_append(qkv, qkv[:, qd:], qkv[:, qd + kd:], q_out, ck, cv, rope, strides, B, Hq, Hkv, 128,
                                          max_seq, 3, S, B, 1e-6, q_in_row_stride=qd + 2 * kd, kv_in_row_stride=qd + 2 * kd)
        else:
            ellm_b200.qk_norm_rope_append(qkv[:, :qd].contiguous(), qkv[:, qd:qd + kd].contiguous(), qkv[:, qd + kd:].contiguous(),
                                          q_out, ck, cv, rope, strides, B, Hq, Hkv, 128, max_seq, 3, S, B, 1e-6)
        torch.cuda.synchronize()
        outs.append((q_out, ck, cv))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    assert outs[0][1].abs().sum() > 0


def test_positions_past_the_rope_table_leave_q_k_and_v_untouched():
    """Per-sequence device positions cannot be validated on the host: a position that is inside the
    cache but has no row in the rotation table must leave the token's whole cache line (K and V)
    and its Q output as they were, never a new V beside a stale K.  In-place x == y of the
    row norm gives the bits of the out-of-place call."""
    dev = torch.device("cuda:0")
    B, Hq, Hkv, max_seq, rope_rows = 3, 4, 2, 64, 16
    g = torch.Generator().manual_seed(11)
    q = torch.randn(1, B, Hq, 128, generator=g).to(torch.bfloat16).to(dev)
    k = torch.randn(1, B, Hkv, 128, generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn(1, B, Hkv, 128, generator=g).to(torch.bfloat16).to(dev)
    rope = torch.from_numpy(ellm_b200.precompute_freqs_cis(128, rope_rows, 1e6)).to(dev)
    strides = [Hkv * max_seq * 128, max_seq * 128, 128, 1]
    ck = torch.full((B, Hkv, max_seq, 128), 7.0, dtype=torch.bfloat16, device=dev)
    cv = torch.full_like(ck, 9.0)
    q_out = torch.full_like(q, 5.0)
    pos = torch.tensor([3, 40, 15], dtype=torch.int32, device=dev)   # sequence 1 lies past the 16 table rows
    ellm_b200.qk_norm_rope_append(q, k, v, q_out, ck, cv, rope, strides, B, Hq, Hkv, 128, max_seq, 0, 1, B, 1e-6,
                                  positions=pos)
    torch.cuda.synchronize()
    assert (ck[1] == 7.0).all() and (cv[1] == 9.0).all() and (q_out[0, 1] == 5.0).all()
    for b, p_ in ((0, 3), (2, 15)):
        assert torch.equal(cv[b, :, p_], v[0, b]) and not (ck[b, :, p_] == 7.0).all() and not (q_out[0, b] == 5.0).all()
        untouched = torch.ones(max_seq, dtype=torch.bool, device=dev)
        untouched[p_] = False
        assert (ck[b][:, untouched] == 7.0).all() and (cv[b][:, untouched] == 9.0).all()
    x = (torch.randn(6, 512, generator=g) * 2).to(torch.bfloat16).to(dev)
    y = torch.zeros_like(x)
    ellm_b200.rms_norm(x, y, 1e-6)
    ellm_b200.rms_norm(x, x, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(x, y)
