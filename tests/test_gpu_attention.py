"""Parity of the CUDA attention path with the CPU oracle, through the C ABI.

Every test here needs a B200.  Inputs are seeded; cache rows past each
sequence's end are NaN so that any out-of-range read poisons the output."""
import numpy as np
import pytest
import torch

import ellm_b200
import oracle
from ellm_b200 import _lib as L
from helpers import Case, assert_attention_close, assert_cache_bit_exact, bits

pytestmark = pytest.mark.gpu


def _check(case, **gpu_kw):
    want_k, want_v, want_o, want_l = case.oracle()
    got_k, got_v, got_o, got_l = case.gpu(**gpu_kw)
    assert_cache_bit_exact(got_k, got_v, want_k, want_v)
    return assert_attention_close(case, got_o, got_l, want_o, want_l)


def test_reference_kat_all_ones_through_the_abi():
    # the reference's only attention KAT (generic/flash_attention.rs:119-147) on the GPU:
    # q = K = V = 1, 8 keys, scale 1 -> O = 1, LSE = 128 + ln 8
    dev = torch.device("cuda:0")
    q = torch.ones(1, 1, 1, 128, dtype=torch.bfloat16, device=dev)
    k = torch.ones(1, 1, 8, 128, dtype=torch.bfloat16, device=dev)
    v = torch.ones(1, 1, 8, 128, dtype=torch.bfloat16, device=dev)
    out = torch.zeros_like(q)
    lse = torch.zeros(1, 1, 1, dtype=torch.float32, device=dev)
    op = ellm_b200.Attention.new(q, k, v, out, 1, 1, 1, 128, [8 * 128, 8 * 128, 128, 1], 1.0, max_seq=8, lse=lse)
    op.run(7, 1, 1, 1, 0)
    assert (out.float() == 1.0).all()
    assert abs(lse.item() - (128.0 + np.log(8.0))) < 1e-3
    assert op.kernel_stats()["decode_splitkv"][0] == 1


@pytest.mark.parametrize("lens", [[1], [2], [63], [64], [65], [127, 128, 129], [1, 700, 64, 3000]])
@pytest.mark.parametrize("q_heads,kv_heads", [(8, 1), (4, 4), (32, 4)])
def test_decode_ragged(lens, q_heads, kv_heads):
    # sequence b holds lens[b]-1 cached tokens; the new token is appended at lens[b]-1
    pos = [n - 1 for n in lens]
    case = Case(seed=100 + len(lens), interval=1, batch=len(lens), q_heads=q_heads, kv_heads=kv_heads,
                max_seq=max(lens) + 3, positions=pos)
    _check(case)
    # two launches per decode step: the append rides in the decode kernel, then the merge
    assert case.last_stats["decode_splitkv"][0] == 1 and case.last_stats["merge"][0] == 1
    assert case.last_stats["kv_append"][0] == 0


def test_decode_uniform_position_and_dead_batch_slots():
    case = Case(seed=7, interval=1, batch=3, max_batch=5, q_heads=16, kv_heads=2, max_seq=300, position_index=257)
    _check(case, cpu_num=4)  # all four thread ids call run; exactly one launches
    assert case.last_stats["decode_splitkv"][0] == 1


def test_decode_wide_group_uses_two_head_tiles():
    case = Case(seed=8, interval=1, batch=2, q_heads=24, kv_heads=1, max_seq=200, positions=[150, 31])
    _check(case)


@pytest.mark.parametrize("group", [1, 2, 3, 5, 7, 8, 9, 12, 15, 16, 17, 33])
def test_decode_every_group_size(group):
    """The decode kernel puts a segment's query heads in blocks of 8 on the N side of its products (one
    block for groups up to 8, two for 9-16, several segments above 16): every fill of the blocks, with
    two KV heads so that a segment's heads are not the tensor's first, against the oracle."""
    case = Case(seed=400 + group, interval=1, batch=3, q_heads=2 * group, kv_heads=2, max_seq=700,
                positions=[699, 64, 200], poison=True)
    _check(case)


@pytest.mark.parametrize("positions", [[20000, 3000], [30000, 10], [9000], [700, 650, 600, 580]])
def test_decode_few_segments_split_by_segment(positions):
    """Steps with few segments snap the decode grid's CTA boundaries to the segment boundaries (one piece
    per CTA) and the merge kernel derives the same ranges: two ragged sequences (every segment gets CTAs of
    its own), a long and a one-tile sequence (the short one's segments would get no CTA: back to the even
    split), one sequence, and four short ones (fewer tiles than CTAs: even split)."""
    case = Case(seed=500 + len(positions), interval=1, batch=len(positions), q_heads=32, kv_heads=4,
                max_seq=max(positions) + 2, positions=positions)
    _check(case)


def test_decode_long_contexts_many_pieces():
    # enough tiles that every CTA gets a piece and sequences span several CTAs
    case = Case(seed=9, interval=1, batch=4, q_heads=32, kv_heads=4, max_seq=8192,
                positions=[8000, 1023, 4097, 6000], poison=True)
    _check(case)


@pytest.mark.parametrize("interval,position_index", [(2, 0), (63, 0), (64, 0), (65, 0), (127, 0), (129, 0), (17, 40), (64, 64)])
@pytest.mark.parametrize("q_heads,kv_heads", [(4, 4), (8, 1), (6, 2)])
def test_prefill_warp_mma_shapes(interval, position_index, q_heads, kv_heads):
    case = Case(seed=200 + interval, interval=interval, batch=2, q_heads=q_heads, kv_heads=kv_heads,
                max_seq=position_index + interval + 5, position_index=position_index)
    _check(case, prefill_kernel=L.PREFILL_WARP_MMA)
    assert case.last_stats["prefill_warp_mma"][0] == 1


def test_prefill_ragged_positions():
    case = Case(seed=21, interval=33, batch=3, q_heads=8, kv_heads=2, max_seq=200, positions=[0, 100, 37])
    _check(case, prefill_kernel=L.PREFILL_WARP_MMA)


def test_chunked_prefill_equals_one_shot():
    """position_index > 0: prefill in chunks of 48 gives the same rows as one pass of 144."""
    dev = torch.device("cuda:0")
    S, Hq, Hkv, chunk = 144, 8, 2, 48
    full = Case(seed=33, interval=S, batch=1, q_heads=Hq, kv_heads=Hkv, max_seq=S, position_index=0, poison=False)
    _, _, want_o, want_l = full.oracle()
    strides = full.strides
    ck = torch.full((1, Hkv, S, 128), float("nan"), dtype=torch.bfloat16, device=dev)
    cv = torch.full_like(ck, float("nan"))
    q = torch.zeros(chunk, 1, Hq, 128, dtype=torch.bfloat16, device=dev)
    kn = torch.zeros(chunk, 1, Hkv, 128, dtype=torch.bfloat16, device=dev)
    vn = torch.zeros_like(kn)
    out = torch.zeros_like(q)
    lse = torch.zeros(chunk, 1, Hq, dtype=torch.float32, device=dev)
    op = ellm_b200.Attention.new(q, ck, cv, out, 1, Hq, Hkv, 128, strides, full.scale, max_seq=S,
                                 max_interval=chunk, lse=lse, k_new=kn, v_new=vn, prefill_kernel=L.PREFILL_WARP_MMA)
    got_o, got_l = [], []
    for p0 in range(0, S, chunk):
        q.copy_(full.q[p0:p0 + chunk]); kn.copy_(full.k_new[p0:p0 + chunk]); vn.copy_(full.v_new[p0:p0 + chunk])
        op.run(p0, chunk, 1, 1, 0)
        got_o.append(bits(out).copy()); got_l.append(lse.cpu().numpy().copy())
    assert_attention_close(full, np.concatenate(got_o), np.concatenate(got_l), want_o, want_l)
    assert np.array_equal(bits(ck).reshape(Hkv, S, 128), bits(full.k_new).reshape(S, Hkv, 128).transpose(1, 0, 2))


def test_run_host_copies_in_and_out():
    case = Case(seed=40, interval=1, batch=3, q_heads=8, kv_heads=2, max_seq=500, positions=[499, 10, 255])
    _check(case, use_run_host=True)
    case = Case(seed=41, interval=20, batch=2, max_batch=3, q_heads=8, kv_heads=2, max_seq=64, position_index=5)
    _check(case, use_run_host=True, prefill_kernel=L.PREFILL_WARP_MMA)


def test_bound_host_step_equals_run_host():
    """Attention.bind_host converts the host-buffer arguments once; the callable it returns is run_host."""
    dev = torch.device("cuda:0")
    case = Case(seed=61, interval=1, batch=3, q_heads=8, kv_heads=2, max_seq=600, positions=[599, 10, 300])
    want_k, want_v, want_o, want_l = case.oracle()
    q, ck, cv = case.q.to(dev), case.cache_k.to(dev), case.cache_v.to(dev)
    out = torch.zeros_like(q)
    lse = torch.zeros(1, case.max_batch, case.q_heads, dtype=torch.float32, device=dev)
    op = ellm_b200.Attention.new(q, ck, cv, out, case.max_batch, case.q_heads, case.kv_heads, 128, case.strides, case.scale,
                                 max_seq=case.max_seq, lse=lse, k_new=torch.zeros_like(case.k_new).to(dev),
                                 v_new=torch.zeros_like(case.v_new).to(dev))
    qh, kh, vh = case.q.clone().pin_memory(), case.k_new.clone().pin_memory(), case.v_new.clone().pin_memory()
    oh = torch.zeros_like(qh).pin_memory()
    lh = torch.zeros(1, case.max_batch, case.q_heads, dtype=torch.float32).pin_memory()
    ph = torch.from_numpy(case.positions).clone().pin_memory()
    step = op.bind_host(qh, oh, 0, 1, case.batch, k_new_host=kh, v_new_host=vh, lse_host=lh, positions_host=ph)
    for _ in range(3):
        oh.zero_()
        step()
    assert_attention_close(case, bits(oh), lh.numpy(), want_o, want_l)
    assert np.array_equal(bits(ck), want_k) and np.array_equal(bits(cv), want_v)
    op.close()


def test_kv_append_standalone_bit_exact_with_canaries():
    dev = torch.device("cuda:0")
    case = Case(seed=50, interval=3, batch=2, max_batch=4, q_heads=2, kv_heads=2, max_seq=16, positions=[0, 13], poison=False)
    want_k, _, _, _ = case.oracle()
    ck = case.cache_k.to(dev)
    ellm_b200.kv_append(ck, case.k_new.to(dev), case.strides, 4, 2, 128, 16, 0, 3, 2,
                        positions=torch.tensor([0, 13], dtype=torch.int32, device=dev))
    torch.cuda.synchronize()
    assert np.array_equal(bits(ck), want_k)


def test_merge_partials_against_oracle():
    import oracle
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(60)
    parts, rows = 5, 37
    o = torch.randn(parts, rows, 128, generator=g)
    l = torch.randn(parts, rows, generator=g) * 3
    l[2, 5] = float("-inf")   # a part that saw no key
    l[:, 9] = float("-inf")   # a row no part saw
    want_o, want_l = oracle.merge_partials(o.numpy(), l.numpy())
    out = torch.zeros(rows, 128, dtype=torch.bfloat16, device=dev)
    lse = torch.zeros(rows, dtype=torch.float32, device=dev)
    ellm_b200.merge_partials(o.to(dev), l.to(dev), out, lse)
    torch.cuda.synchronize()
    keep = np.ones(rows, bool); keep[9] = False
    assert np.abs(out.float().cpu().numpy()[keep] - want_o[keep]).max() < 2e-2
    assert np.abs(lse.cpu().numpy()[keep] - want_l[keep]).max() < 1e-4
    assert (out[9] == 0).all() and lse[9].item() == float("-inf")


def test_split_window_partials_merge_to_the_full_result():
    """Key windows [0,a), [a,b), [b,inf) merged == unsplit: decode and prefill."""
    dev = torch.device("cuda:0")
    for interval, pos in ((1, 700), (40, 300)):
        case = Case(seed=70 + interval, interval=interval, batch=2, q_heads=8, kv_heads=2, max_seq=pos + interval,
                    position_index=pos, poison=False)
        want_k, want_v, want_o, want_l = case.oracle()
        q = case.q.to(dev)
        ck, cv = from_bits_dev(want_k, case, dev), from_bits_dev(want_v, case, dev)
        out = torch.zeros_like(q)
        op = ellm_b200.Attention.new(q, ck, cv, out, 2, 8, 2, 128, case.strides, case.scale, max_seq=case.max_seq,
                                     max_interval=interval, prefill_kernel=L.PREFILL_WARP_MMA)
        windows = [(0, 100), (100, 333), (333, 1 << 40)]
        po = torch.zeros(len(windows), interval, 2, 8, 128, dtype=torch.float32, device=dev)
        pl = torch.zeros(len(windows), interval, 2, 8, dtype=torch.float32, device=dev)
        for i, (a, b) in enumerate(windows):
            op.run_window(pos, interval, 2, a, b, po[i], pl[i])
        rows = interval * 2 * 8
        lse = torch.zeros(rows, dtype=torch.float32, device=dev)
        ellm_b200.merge_partials(po.view(len(windows), rows, 128), pl.view(len(windows), rows), out, lse)
        torch.cuda.synchronize()
        assert_attention_close(case, bits(out), lse.view(interval, 2, 8).cpu().numpy(), want_o, want_l)


def from_bits_dev(a, case, dev):
    from helpers import from_bits
    return from_bits(a).view(case.max_batch, case.kv_heads, case.max_seq, 128).to(dev)


def test_error_paths_on_a_live_handle():
    dev = torch.device("cuda:0")
    q = torch.zeros(1, 2, 4, 128, dtype=torch.bfloat16, device=dev)
    k = torch.zeros(2, 2, 16, 128, dtype=torch.bfloat16, device=dev)
    out = torch.zeros_like(q)
    op = ellm_b200.Attention.new(q, k, k.clone(), out, 2, 4, 2, 128, [2 * 16 * 128, 16 * 128, 128, 1], 0.1, max_seq=16)
    with pytest.raises(ellm_b200.EllmError) as e:
        op.run(16, 1, 1, 1, 0)          # position past max_seq
    assert e.value.status == L.ERR_INVALID_ARG
    with pytest.raises(ellm_b200.EllmError):
        op.run(0, 1, 3, 1, 0)           # batch > max_batch
    with pytest.raises(ellm_b200.EllmError):
        op.run(0, 2, 1, 1, 0)           # interval > max_interval
    with pytest.raises(ellm_b200.EllmError):
        op.run(0, 1, 1, 2, 2)           # thread_id outside cpu_num
    op.run(3, 1, 2, 8, 5)               # a non-zero thread id is a no-op
    assert op.kernel_stats()["decode_splitkv"][0] == 0
    op.run(3, 1, 2, 8, 0)
    assert op.kernel_stats()["decode_splitkv"][0] == 1


def test_run_host_replays_its_graph_with_new_contents():
    """Decode through host buffers, three steps with the same page-locked buffers and different
    contents (and advancing positions): every step matches the oracle."""
    import oracle
    from helpers import O_MAX_ABS, LSE_MAX_ABS
    dev = torch.device("cuda:0")
    B, Hq, Hkv, max_seq = 3, 8, 2, 400
    g = torch.Generator().manual_seed(123)
    ck = torch.randn(B, Hkv, max_seq, 128, generator=g).to(torch.bfloat16)
    cv = torch.randn(B, Hkv, max_seq, 128, generator=g).to(torch.bfloat16)
    strides = [Hkv * max_seq * 128, max_seq * 128, 128, 1]
    dq = torch.zeros(1, B, Hq, 128, dtype=torch.bfloat16, device=dev)
    dkn = torch.zeros(1, B, Hkv, 128, dtype=torch.bfloat16, device=dev)
    dvn = torch.zeros_like(dkn)
    dout = torch.zeros_like(dq)
    dlse = torch.zeros(1, B, Hq, dtype=torch.float32, device=dev)
    dck, dcv = ck.to(dev), cv.to(dev)
    op = ellm_b200.Attention.new(dq, dck, dcv, dout, B, Hq, Hkv, 128, strides, 0.0884, max_seq=max_seq, lse=dlse, k_new=dkn, v_new=dvn)
    qh = torch.zeros(1, B, Hq, 128, dtype=torch.bfloat16).pin_memory()
    knh = torch.zeros(1, B, Hkv, 128, dtype=torch.bfloat16).pin_memory()
    vnh = torch.zeros_like(knh).pin_memory()
    oh = torch.zeros_like(qh).pin_memory()
    lh = torch.zeros(1, B, Hq, dtype=torch.float32).pin_memory()
    ph = torch.tensor([10, 200, 57], dtype=torch.int32).pin_memory()
    ref_k, ref_v = bits(ck).copy(), bits(cv).copy()
    for step in range(3):
        qh.copy_(torch.randn(1, B, Hq, 128, generator=g).to(torch.bfloat16))
        knh.copy_(torch.randn(1, B, Hkv, 128, generator=g).to(torch.bfloat16))
        vnh.copy_(torch.randn(1, B, Hkv, 128, generator=g).to(torch.bfloat16))
        op.run_host(qh, oh, 0, 1, B, k_new_host=knh, v_new_host=vnh, lse_host=lh, positions_host=ph)
        pos = ph.numpy().copy()
        for cache, new in ((ref_k, knh), (ref_v, vnh)):
            oracle.kv_append_bf16(cache, bits(new), strides, B, Hkv, 128, 0, 1, B, positions=pos)
        want_o, want_l = oracle.attention_bf16(bits(qh), ref_k, ref_v, strides, Hq, Hkv, 0.0884, 0, 1, B, positions=pos)
        assert np.abs(oh.float().numpy() - oracle.bf16_bits_to_f32(want_o)).max() <= O_MAX_ABS
        assert np.abs(lh.numpy() - want_l).max() <= LSE_MAX_ABS
        ph += 1
    assert np.array_equal(bits(dck), ref_k) and np.array_equal(bits(dcv), ref_v)
    assert op.kernel_stats()["decode_splitkv"][0] == 3


@pytest.mark.parametrize("ctas", [1, 37, 148])
def test_decode_grid_size_option(ctas):
    """The decode kernel splits its tile list over any number of CTAs up to 2 x SMs (option
    "decode_ctas"); the result does not depend on the split beyond the merge's rounding."""
    import oracle
    from helpers import O_MAX_ABS, LSE_MAX_ABS
    dev = torch.device("cuda:0")
    case = Case(seed=31, interval=1, batch=3, q_heads=8, kv_heads=2, max_seq=3000, positions=[2999, 65, 1500])
    want_k, want_v, want_o, want_l = case.oracle()
    q, ck, cv = case.q.to(dev), case.cache_k.to(dev), case.cache_v.to(dev)
    out = torch.zeros_like(q)
    lse = torch.zeros(1, case.max_batch, case.q_heads, dtype=torch.float32, device=dev)
    op = ellm_b200.Attention.new(q, ck, cv, out, case.max_batch, case.q_heads, case.kv_heads, 128, case.strides, case.scale,
                                 max_seq=case.max_seq, lse=lse, k_new=case.k_new.to(dev), v_new=case.v_new.to(dev))
    op.set_option("decode_ctas", ctas)
    op.run_ragged(torch.from_numpy(case.positions).to(dev), 1, case.batch)
    assert np.array_equal(bits(ck), want_k) and np.array_equal(bits(cv), want_v)
    assert np.abs(out.float().cpu().numpy() - oracle.bf16_bits_to_f32(want_o))[:, :case.batch].max() <= O_MAX_ABS
    assert np.abs(lse.cpu().numpy() - want_l)[:, :case.batch].max() <= LSE_MAX_ABS
    with pytest.raises(ellm_b200.EllmError):
        op.set_option("decode_ctas", 100000)
    op.close()


@pytest.mark.parametrize("fused_append", [False, True])
def test_decode_with_early_streaming_matches_the_oracle(fused_append):
    """decode_early_stream: the decode kernel requests its first K/V rows before it waits for the
    stream's previous kernel.  Steps are enqueued back to back (each step's merge still reads one
    copy of the partials while the next step's decode kernel fills the other), with the positions
    advancing between steps from the host side; every step is compared with the oracle.  Short and
    long sequences, so that some CTAs' first stage holds a newest row (which must not be read early)."""
    dev = torch.device("cuda:0")
    B, Hq, Hkv, max_seq, steps = 5, 16, 2, 4200, 4
    base = np.array([4100, 0, 63, 2047, 130], dtype=np.int32)
    g = torch.Generator().manual_seed(99)
    full_k = torch.randn(B, Hkv, max_seq, 128, generator=g).to(torch.bfloat16)
    full_v = torch.randn(B, Hkv, max_seq, 128, generator=g).to(torch.bfloat16)
    qs = torch.randn(steps, 1, B, Hq, 128, generator=g).to(torch.bfloat16)
    ck, cv = full_k.clone().to(dev), full_v.clone().to(dev)
    if fused_append:   # rows from each sequence's start position on arrive step by step through k_new / v_new
        for b in range(B):
            ck[b, :, base[b]:] = float("nan")
            cv[b, :, base[b]:] = float("nan")
    q = torch.zeros(1, B, Hq, 128, dtype=torch.bfloat16, device=dev)
    kn = torch.zeros(1, B, Hkv, 128, dtype=torch.bfloat16, device=dev)
    vn = torch.zeros_like(kn)
    outs = torch.zeros(steps, 1, B, Hq, 128, dtype=torch.bfloat16, device=dev)
    lses = torch.zeros(steps, 1, B, Hq, dtype=torch.float32, device=dev)
    pos_all = torch.from_numpy(np.stack([base + s for s in range(steps)])).to(dev)
    ops = [ellm_b200.Attention.new(q, ck, cv, outs[s], B, Hq, Hkv, 128, [Hkv * max_seq * 128, max_seq * 128, 128, 1], 0.088,
                                   max_seq=max_seq, lse=lses[s], k_new=kn if fused_append else None,
                                   v_new=vn if fused_append else None, async_=True, early_stream=True) for s in range(steps)]
    for s in range(steps):
        # the step's inputs are staged by plain stream-ordered copies (not programmatic dependents), so
        # they are complete before the decode kernel can start
        q.copy_(qs[s].to(dev))
        if fused_append:
            for b in range(B):
                kn[0, b].copy_(full_k[b, :, base[b] + s].to(dev))
                vn[0, b].copy_(full_v[b, :, base[b] + s].to(dev))
        ops[s].run_ragged(pos_all[s], 1, B, 1, 0)
        ops[s].run_ragged(pos_all[s], 1, B, 1, 0)     # the same step again, back to back: kernel after kernel
    torch.cuda.synchronize()
    for op in ops:
        op.check()
        op.close()
    strides = [Hkv * max_seq * 128, max_seq * 128, 128, 1]
    for s in range(steps):
        want_o, want_l = oracle.attention_bf16(bits(qs[s]), bits(full_k), bits(full_v), strides, Hq, Hkv, 0.088, 0, 1, B,
                                               max_batch=B, positions=base + s)
        d = np.abs(outs[s].float().cpu().numpy() - oracle.bf16_bits_to_f32(want_o))
        assert np.isfinite(d).all() and d.max() <= 2e-2 and d.mean() <= 2e-3, (s, d.max())
        assert np.abs(lses[s].cpu().numpy() - want_l).max() <= 1e-3
    if fused_append:
        for b in range(B):
            assert torch.equal(ck[b, :, base[b]:base[b] + steps].cpu(), full_k[b, :, base[b]:base[b] + steps])
            assert torch.isnan(ck[b, :, base[b] + steps:].float()).all()
