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


def test_config5_prefix_65536_through_the_chunk_window_and_merge_path():
    """BASELINE configs[4]'s own check: the first 65536 tokens of the seed-4 sequence (one KV-head
    group, 8 query heads / 1 KV head; the tensors are generated at the full 1048576 length and
    sliced), cut into 8 zig-zag chunks over 4 emulated ranks and pushed through the steps of
    sharding.sequence_chunk_attention one rank after the other on one GPU - ellm_attn_run_window_q
    per (query chunk, key chunk) pair on a chunk-local cache, the local pre-merge, the hand-over of
    the partials to the chunk's owner, the final ellm_attn_merge_partials_list - and 576 sampled
    rows, spread over every chunk and on both sides of every chunk edge, are recomputed by the
    oracle's row kernel over all their keys."""
    from concurrent.futures import ThreadPoolExecutor
    from ellm_b200 import merge_partials_list, sharding
    dev = torch.device("cuda:0")
    S_full, S, G, world = 1048576, 65536, 8, 4
    gen = torch.Generator(device=dev).manual_seed(4)
    q = torch.randn(S_full, 1, G, 128, device=dev, generator=gen).to(torch.bfloat16)[:S].contiguous()
    k = torch.randn(1, 1, S_full, 128, device=dev, generator=gen).to(torch.bfloat16)[:, :, :S].contiguous()
    v = torch.randn(1, 1, S_full, 128, device=dev, generator=gen).to(torch.bfloat16)[:, :, :S].contiguous()
    scale = 1.0 / np.sqrt(128.0)
    plan = sharding.SequenceChunkPlan(seq_len=S, world=world, zigzag=True)
    Lc, n = plan.chunk_len, plan.n_chunks
    q_all = q.view(n, Lc, 1, G, 128)
    dummy = torch.empty(Lc, 1, G, 128, dtype=torch.bfloat16, device=dev)
    ops = {}
    for c in range(n):   # every chunk's K/V rows as their owner holds them: a chunk-local cache
        kc, vc = k[:, :, c * Lc:(c + 1) * Lc].contiguous(), v[:, :, c * Lc:(c + 1) * Lc].contiguous()
        ops[c] = (ellm_b200.Attention.new(q_all[0], kc, vc, dummy, 1, G, 1, 128, [Lc * 128, Lc * 128, 128, 1], scale,
                                          max_seq=Lc, max_interval=Lc, async_=True), kc, vc)

    def new_partial():
        return (torch.empty(Lc, 1, G, 128, dtype=torch.float32, device=dev),
                torch.empty(Lc, 1, G, dtype=torch.float32, device=dev))

    def compute_partial(i, kc):
        o, lse = new_partial()
        ops[kc][0].run_window_q(q_all[i], (i - kc) * Lc, Lc, 1, 0, Lc, o, lse)
        return o, lse

    def merge(parts):
        o, lse = new_partial()
        merge_partials_list([p[0] for p in parts], [p[1] for p in parts], o, lse, out_f32=True)
        return o, lse

    local = {r: sharding.local_partials(plan, r, compute_partial, merge) for r in range(world)}
    result = {}
    for r in range(world):
        received = {i: [local[src][i] for src in plan.sources_of(i) if src != r] for i in plan.chunks_of(r)}
        result.update(sharding.final_merge(plan, r, local[r], received, merge))
    for op, _, _ in ops.values():
        op.check()
    assert sorted(result) == list(range(n))
    assert sum(len(plan.sources_of(i)) > 1 for i in range(n)) >= n - 1   # all but chunk 0 pass through the merge

    rng = np.random.default_rng(65536)
    rows = set()
    for c in range(n):
        rows.update([c * Lc, c * Lc + 1, c * Lc + 127, c * Lc + 128, (c + 1) * Lc - 129, (c + 1) * Lc - 2, (c + 1) * Lc - 1])
        rows.update(int(x) for x in rng.integers(c * Lc, (c + 1) * Lc, 65))
    rows = sorted(rows)
    assert len(rows) >= 512
    kf, vf = k[0, 0].float().cpu().numpy(), v[0, 0].float().cpu().numpy()
    got = {}
    for idx, r in enumerate(rows):
        c, rr, h = r // Lc, r % Lc, idx % G
        got[r] = (q[r, 0, h].float().cpu().numpy(), result[c][0][rr, 0, h].cpu().numpy(), float(result[c][1][rr, 0, h]), h)

    def one(r):
        qf, go, gl, h = got[r]
        o = np.zeros(128, np.float32)
        want_l = oracle.flash_attention_f32(qf, kf, vf, o, scale, r)
        return float(np.abs(go - o).max()), float(np.abs(go - o).mean()), abs(gl - want_l)

    with ThreadPoolExecutor(8) as pool:
        res = list(pool.map(one, rows))
    assert max(x[0] for x in res) <= O_MAX_ABS, max(x[0] for x in res)
    assert np.mean([x[1] for x in res]) <= O_MEAN_ABS
    assert max(x[2] for x in res) <= LSE_MAX_ABS, max(x[2] for x in res)
    for op, _, _ in ops.values():
        op.close()


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


def test_config4_layer_projections_full_chunk_sampled_rows():
    """BASELINE configs[3]'s layer shape at its full prefill chunk (32768 rows, hidden 2048, 32 q / 4 kv
    heads): the fused QKV projection and the output projection with residual run at full size (CTA pairs),
    and 96 sampled rows - the first and last of the chunk, tile edges, random ones - are compared with the
    oracle, which only needs those rows of A.  A second run with one CTA per tile must give the same bits
    on every row (the two forms add the same products in the same order)."""
    from ellm_b200.projection import MatMul3, MatMulAdd
    dev = torch.device("cuda:0")
    S, hidden, Hq, Hkv = 32768, 2048, 32, 4
    qd, kd = Hq * 128, Hkv * 128
    g = torch.Generator().manual_seed(3)
    x = torch.randn(S, hidden, generator=g).to(torch.bfloat16)
    wqkv = (torch.randn(qd + 2 * kd, hidden, generator=g) * 0.02).to(torch.bfloat16)
    wo = (torch.randn(hidden, qd, generator=g) * 0.02).to(torch.bfloat16)
    qw = (1 + 0.02 * torch.randn(128, generator=g)).float()
    kw = (1 + 0.02 * torch.randn(128, generator=g)).float()
    rope = ellm_b200.precompute_freqs_cis(128, S, 1e6)
    strides = [Hkv * S * 128, S * 128, 128, 1]
    rows = np.unique(np.concatenate([[0, 1, 127, 128, 255, 256, S - 257, S - 256, S - 129, S - 128, S - 1],
                                     np.random.default_rng(4).integers(0, S, 85)]))
    dx, dw, dwo = x.to(dev), wqkv.to(dev), wo.to(dev)
    results = []
    for pairing in (-1, 0):
        ck = torch.zeros(1, Hkv, S, 128, dtype=torch.bfloat16, device=dev)
        cv = torch.zeros_like(ck)
        q = torch.zeros(S, 1, Hq, 128, dtype=torch.bfloat16, device=dev)
        y = dx.clone()
        op3 = MatMul3.new(dx, dw[:qd], q, dw[qd:qd + kd], ck, dw[qd + kd:], cv, torch.from_numpy(rope).to(dev), 128, S, hidden,
                          qd, kd, kv_strides=strides, max_batch=1, max_seq=S, rope_rows=S, q_norm_weight=qw.to(dev),
                          k_norm_weight=kw.to(dev))
        op3.set_pairing(pairing)
        op3.run(0, S, 1)
        a = q.view(S, qd)   # any bf16 matrix serves as the output projection's input
        opa = MatMulAdd.new(a, dwo, y, y, S, hidden, qd, max_batch=1)
        opa.set_pairing(pairing)
        opa.run(0, S, 1)
        results.append((bits(q), bits(ck), bits(cv), bits(y)))
        op3.close()
        opa.close()
    for u, v in zip(*results):
        assert np.array_equal(u, v)
    gq, gk, gv, gy = results[0]
    # oracle on the sampled rows only: each row is the token at position = its index
    xs = bits(x)[rows]
    pq = oracle.matmul_nt_bf16(xs, bits(wqkv)[:qd]).reshape(len(rows), 1, Hq, 128)
    pk = oracle.matmul_nt_bf16(xs, bits(wqkv)[qd:qd + kd]).reshape(len(rows), 1, Hkv, 128)
    pv = oracle.matmul_nt_bf16(xs, bits(wqkv)[qd + kd:]).reshape(len(rows), 1, Hkv, 128)
    for i, r in enumerate(rows):
        ck1 = np.zeros((1, Hkv, S, 128), np.uint16) if i == 0 else ck1
        cv1 = np.zeros((1, Hkv, S, 128), np.uint16) if i == 0 else cv1
        wq_row = oracle.qk_norm_rope_append_bf16(pq[i:i + 1], pk[i:i + 1], pv[i:i + 1], ck1, cv1, rope, strides, Hq, Hkv,
                                                 int(r), 1, 1, 1e-6, q_weight=qw.numpy(), k_weight=kw.numpy())
        gw, ww = oracle.bf16_bits_to_f32(gq[r]), oracle.bf16_bits_to_f32(wq_row[0])
        assert (gq[r] == wq_row[0]).mean() >= 0.95 and np.abs(gw - ww).max() <= 2.0 ** -5
    for name, got, want in (("k", gk, ck1), ("v", gv, cv1)):
        g32, w32 = oracle.bf16_bits_to_f32(got[0][:, rows]), oracle.bf16_bits_to_f32(want[0][:, rows])
        assert (got[0][:, rows] == want[0][:, rows]).mean() >= 0.97, name
        assert np.abs(g32 - w32).max() <= 2.0 ** -5, name
    want_y = oracle.matmul_nt_bf16(gq.reshape(S, qd)[rows], bits(wo), bits(x)[rows])
    g32, w32 = oracle.bf16_bits_to_f32(gy[rows]), oracle.bf16_bits_to_f32(want_y)
    assert (gy[rows] == want_y).mean() >= 0.99
    assert (np.abs(g32 - w32) <= np.abs(w32) * 2.0 ** -7 + 2e-5 * np.sqrt(qd)).all()
