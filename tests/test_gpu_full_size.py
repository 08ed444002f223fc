"""Parity at the benchmark configurations' full sizes (B200 only).

Configurations 1 and 2 are compared with the oracle in full.  The long-sequence
configurations (3: seq 131072, 5: seq 1048576; one KV-head group each, which is what one GPU
owns) are too large for a full CPU pass, so they are checked through properties that do not
depend on size: sampled query rows against the oracle's row kernel over the full key range,
and the tcgen05 kernel against the independent warp-MMA kernel on every row of a 32768 prefix.
"""
import numpy as np
import pytest
import torch

import ellm_b200
import oracle
from ellm_b200 import _lib as L
from helpers import Case, O_MAX_ABS, O_MEAN_ABS, LSE_MAX_ABS, assert_attention_close, assert_cache_bit_exact, bits

pytestmark = pytest.mark.gpu


def test_config1_full_prefill_2048_mha():
    # BASELINE configs[0]: seq 2048, 32 = 32 heads, cache max_seq 4096, seed 0
    case = Case(seed=0, interval=2048, batch=1, q_heads=32, kv_heads=32, max_seq=4096, position_index=0)
    want_k, want_v, want_o, want_l = case.oracle()
    got_k, got_v, got_o, got_l = case.gpu()
    assert case.last_stats["prefill_tcgen05"][0] == 1
    assert_cache_bit_exact(got_k, got_v, want_k, want_v)
    assert_attention_close(case, got_o, got_l, want_o, want_l)


def test_config2_full_decode_16_ragged_sequences():
    # BASELINE configs[1]: 32 q / 4 kv heads, 16 sequences, lens U[1024, 32768] seed 1, max_seq 32768
    g = torch.Generator().manual_seed(1)
    lens = torch.randint(1024, 32769, (16,), generator=g).numpy()
    pos = np.minimum(lens, 32767)   # append at `len`, attend over len + 1 (kept inside the cache)
    case = Case(seed=1, interval=1, batch=16, q_heads=32, kv_heads=4, max_seq=32768, positions=pos)
    want_k, want_v, want_o, want_l = case.oracle()
    got_k, got_v, got_o, got_l = case.gpu()
    assert_cache_bit_exact(got_k, got_v, want_k, want_v)
    assert_attention_close(case, got_o, got_l, want_o, want_l)


def _sampled_rows_check(S, G, rows, seed):
    """One KV-head group (G query heads, 1 KV head), causal prefill of S tokens with the tcgen05
    kernel; the sampled rows are recomputed by the oracle's row kernel over all their keys."""
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(seed)
    q = torch.randn(S, 1, G, 128, device=dev, generator=gen).to(torch.bfloat16)
    k = torch.randn(1, 1, S, 128, device=dev, generator=gen).to(torch.bfloat16)
    v = torch.randn(1, 1, S, 128, device=dev, generator=gen).to(torch.bfloat16)
    out = torch.zeros_like(q)
    lse = torch.zeros(S, 1, G, dtype=torch.float32, device=dev)
    scale = 1.0 / np.sqrt(128.0)
    op = ellm_b200.Attention.new(q, k, v, out, 1, G, 1, 128, [S * 128, S * 128, 128, 1], scale, max_seq=S,
                                 max_interval=S, lse=lse, prefill_kernel=L.PREFILL_TCGEN05)
    op.run(0, S, 1, 1, 0)
    kf = k[0, 0].float().cpu().numpy()
    vf = v[0, 0].float().cpu().numpy()
    worst_o = worst_l = 0.0
    for r in rows:
        for h in range(G):
            qf = q[r, 0, h].float().cpu().numpy()
            o = np.zeros(128, np.float32)
            want_l = oracle.flash_attention_f32(qf, kf, vf, o, scale, r)
            want_o = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(o))
            worst_o = max(worst_o, float(np.abs(out[r, 0, h].float().cpu().numpy() - want_o).max()))
            worst_l = max(worst_l, abs(float(lse[r, 0, h]) - want_l))
    assert worst_o <= O_MAX_ABS, worst_o
    assert worst_l <= LSE_MAX_ABS, worst_l
    return q, k, v, out, lse


def test_config3_one_head_group_seq_131072_sampled_rows():
    S = 131072
    _sampled_rows_check(S, 8, [0, 1, 127, 128, 129, 4095, 65535, 65536, 100000, S - 129, S - 2, S - 1], seed=2)


def test_config5_one_head_group_seq_1048576_sampled_rows():
    S = 1048576
    _sampled_rows_check(S, 8, [0, 255, 256, 65535, 524287, 524288, 1000003, S - 1], seed=4)


def test_tcgen05_and_warp_mma_kernels_agree_on_every_row_at_32768():
    dev = torch.device("cuda:0")
    S, G = 32768, 8
    q, k, v, out_tc, lse_tc = _sampled_rows_check(S, G, [0, 12345, S - 1], seed=5)
    out = torch.zeros_like(q)
    lse = torch.zeros_like(lse_tc)
    op = ellm_b200.Attention.new(q, k, v, out, 1, G, 1, 128, [S * 128, S * 128, 128, 1], 1.0 / np.sqrt(128.0), max_seq=S,
                                 max_interval=S, lse=lse, prefill_kernel=L.PREFILL_WARP_MMA)
    op.run(0, S, 1, 1, 0)
    d = (out.float() - out_tc.float()).abs()
    assert d.max().item() <= O_MAX_ABS and d.mean().item() <= O_MEAN_ABS
    assert (lse - lse_tc).abs().max().item() <= LSE_MAX_ABS
    # chunked prefill (4 chunks with position_index > 0) equals the one-shot pass
    chunk = S // 4
    qc = torch.zeros(chunk, 1, G, 128, dtype=torch.bfloat16, device=dev)
    oc = torch.zeros_like(qc)
    lc = torch.zeros(chunk, 1, G, dtype=torch.float32, device=dev)
    op2 = ellm_b200.Attention.new(qc, k, v, oc, 1, G, 1, 128, [S * 128, S * 128, 128, 1], 1.0 / np.sqrt(128.0), max_seq=S,
                                  max_interval=chunk, lse=lc, prefill_kernel=L.PREFILL_TCGEN05)
    for c in range(4):
        qc.copy_(q[c * chunk:(c + 1) * chunk])
        op2.run(c * chunk, chunk, 1, 1, 0)
        d = (oc.float() - out_tc[c * chunk:(c + 1) * chunk].float()).abs()
        assert d.max().item() <= O_MAX_ABS and d.mean().item() <= O_MEAN_ABS
        assert (lc - lse_tc[c * chunk:(c + 1) * chunk]).abs().max().item() <= LSE_MAX_ABS
