"""Parity of the tcgen05 / TMEM / TMA prefill kernel with the CPU oracle (B200 only)."""
import numpy as np
import pytest
import torch

import ellm_b200
from ellm_b200 import _lib as L
from helpers import Case, assert_attention_close, assert_cache_bit_exact, bits

pytestmark = pytest.mark.gpu


def _check(case):
    want_k, want_v, want_o, want_l = case.oracle()
    got_k, got_v, got_o, got_l = case.gpu(prefill_kernel=L.PREFILL_TCGEN05)
    assert_cache_bit_exact(got_k, got_v, want_k, want_v)
    assert case.last_stats["prefill_tcgen05"][0] == 1 and case.last_stats["prefill_warp_mma"][0] == 0
    return assert_attention_close(case, got_o, got_l, want_o, want_l)


@pytest.mark.parametrize("interval,position_index", [(2, 0), (127, 0), (128, 0), (129, 0), (255, 0), (256, 0), (257, 0),
                                                     (384, 0), (100, 28), (130, 128), (513, 300)])
@pytest.mark.parametrize("q_heads,kv_heads", [(2, 2), (8, 1), (4, 2), (32, 2)])
def test_tcgen05_prefill_shapes(interval, position_index, q_heads, kv_heads):
    case = Case(seed=700 + interval + q_heads, interval=interval, batch=2, q_heads=q_heads, kv_heads=kv_heads,
                max_seq=position_index + interval + 9, position_index=position_index, max_batch=3)
    _check(case)


def test_tcgen05_prefill_llama7b_shape_one_head_group():
    # BASELINE configs[0] geometry (seq 2048, MHA) on 4 of its 32 heads to keep the oracle quick
    case = Case(seed=0, interval=2048, batch=1, q_heads=4, kv_heads=4, max_seq=4096, position_index=0)
    _check(case)


def test_tcgen05_prefill_reference_layout_seq_major_cache():
    """The stride vector the reference model code produces (src/qwen3_moe/attention.rs:149-166):
    K/V physically [seq, batch, kv_head, d], passed as strides [Hkv*D, D, batch*Hkv*D, 1]."""
    dev = torch.device("cuda:0")
    S, B, Hq, Hkv = 200, 2, 8, 2
    case = Case(seed=77, interval=S, batch=B, q_heads=Hq, kv_heads=Hkv, max_seq=S, position_index=0, poison=False)
    _, _, want_o, want_l = case.oracle()
    k_seq_major = case.k_new.to(dev).contiguous()  # [S, B, Hkv, D] is exactly the chunk's rows
    v_seq_major = case.v_new.to(dev).contiguous()
    q = case.q.to(dev)
    out = torch.zeros_like(q)
    lse = torch.zeros(S, B, Hq, dtype=torch.float32, device=dev)
    op = ellm_b200.Attention.new(q, k_seq_major, v_seq_major, out, B, Hq, Hkv, 128, [Hkv * 128, 128, B * Hkv * 128, 1],
                                 case.scale, max_seq=S, max_interval=S, lse=lse, prefill_kernel=L.PREFILL_TCGEN05)
    op.run(0, S, B, 1, 0)
    assert_attention_close(case, bits(out), lse.cpu().numpy(), want_o, want_l)


def test_auto_picks_tcgen05_for_large_chunks_and_warp_mma_for_small():
    big = Case(seed=1, interval=256, batch=1, q_heads=2, kv_heads=2, max_seq=256)
    big.gpu()
    assert big.last_stats["prefill_tcgen05"][0] == 1
    small = Case(seed=1, interval=16, batch=1, q_heads=2, kv_heads=2, max_seq=32)
    small.gpu()   # 16 packed rows per KV head are enough for a tensor-memory tile
    assert small.last_stats["prefill_tcgen05"][0] == 1 and small.last_stats["prefill_warp_mma"][0] == 0
    tiny = Case(seed=1, interval=15, batch=1, q_heads=2, kv_heads=2, max_seq=32)
    tiny.gpu()
    assert tiny.last_stats["prefill_warp_mma"][0] == 1
    ragged = Case(seed=1, interval=256, batch=2, q_heads=2, kv_heads=2, max_seq=600, positions=[0, 300])
    ragged.gpu()   # per-sequence chunk starts stay on the tcgen05 kernel
    assert ragged.last_stats["prefill_tcgen05"][0] == 1


def test_tcgen05_unsupported_group_is_reported():
    dev = torch.device("cuda:0")
    q = torch.zeros(4, 1, 6, 128, dtype=torch.bfloat16, device=dev)
    k = torch.zeros(1, 2, 8, 128, dtype=torch.bfloat16, device=dev)
    with pytest.raises(ellm_b200.EllmError) as e:   # 3 query heads per KV head does not divide 128
        ellm_b200.Attention.new(q, k, k.clone(), torch.zeros_like(q), 1, 6, 2, 128, [2 * 8 * 128, 8 * 128, 128, 1], 0.1,
                                max_seq=8, max_interval=4, prefill_kernel=L.PREFILL_TCGEN05)
    assert e.value.status == L.ERR_UNSUPPORTED


@pytest.mark.parametrize("kernel", [L.PREFILL_TCGEN05, L.PREFILL_WARP_MMA])
def test_sequence_chunks_as_key_windows_merge_to_the_full_result(kernel):
    """What sequence-chunk sharding does, on one GPU: the keys are cut into chunks held in
    separate caches; a query chunk takes an fp32 partial (O, LSE) against each earlier chunk
    (placed past that cache's end, so it sees all of its keys) and a causal one against its
    own; the merged partials equal the unsplit result."""
    dev = torch.device("cuda:0")
    S, Hq, Hkv, chunk = 768, 8, 2, 256
    full = Case(seed=88, interval=S, batch=1, q_heads=Hq, kv_heads=Hkv, max_seq=S, position_index=0, poison=False)
    _, _, want_o, want_l = full.oracle()
    n = S // chunk
    strides = [Hkv * chunk * 128, chunk * 128, 128, 1]
    # chunk caches [1, Hkv, chunk, 128] from the chunk's rows [chunk, 1, Hkv, 128]
    caches = [(full.k_new[c * chunk:(c + 1) * chunk, 0].permute(1, 0, 2).contiguous().to(dev)[None],
               full.v_new[c * chunk:(c + 1) * chunk, 0].permute(1, 0, 2).contiguous().to(dev)[None]) for c in range(n)]
    got_o = np.zeros((S, 1, Hq, 128), np.uint16)
    got_l = np.zeros((S, 1, Hq), np.float32)
    for i in range(n):
        q = full.q[i * chunk:(i + 1) * chunk].contiguous().to(dev)
        po = torch.zeros(i + 1, chunk, 1, Hq, 128, dtype=torch.float32, device=dev)
        pl = torch.zeros(i + 1, chunk, 1, Hq, dtype=torch.float32, device=dev)
        for k in range(i + 1):
            ck, cv = caches[k]
            op = ellm_b200.Attention.new(q, ck, cv, torch.zeros_like(q), 1, Hq, Hkv, 128, strides, full.scale,
                                         max_seq=chunk, max_interval=chunk, prefill_kernel=kernel)
            op.run_window((i - k) * chunk, chunk, 1, 0, chunk, po[k], pl[k])
            name = "prefill_tcgen05" if kernel == L.PREFILL_TCGEN05 else "prefill_warp_mma"
            assert op.kernel_stats()[name][0] == 1
            op.close()
        out = torch.zeros(chunk * Hq, 128, dtype=torch.bfloat16, device=dev)
        lse = torch.zeros(chunk * Hq, dtype=torch.float32, device=dev)
        ellm_b200.merge_partials(po.view(i + 1, chunk * Hq, 128), pl.view(i + 1, chunk * Hq), out, lse)
        torch.cuda.synchronize()
        got_o[i * chunk:(i + 1) * chunk] = bits(out).reshape(chunk, 1, Hq, 128)
        got_l[i * chunk:(i + 1) * chunk] = lse.cpu().numpy().reshape(chunk, 1, Hq)
    assert_attention_close(full, got_o, got_l, want_o, want_l)


@pytest.mark.parametrize("positions,interval", [([0, 300, 37], 200), ([5, 0], 128), ([1000, 1, 511, 512], 129), ([0], 256)])
@pytest.mark.parametrize("q_heads,kv_heads", [(8, 2), (4, 4)])
def test_tcgen05_prefill_per_sequence_chunk_starts(positions, interval, q_heads, kv_heads):
    """Sequences of a batch at different positions; the cache past every sequence's end is NaN, so a
    V row read past the end without being cleared would poison the output."""
    case = Case(seed=900 + interval, interval=interval, batch=len(positions), q_heads=q_heads, kv_heads=kv_heads,
                max_seq=max(positions) + interval + 70, positions=positions, max_batch=len(positions) + 1)
    _check(case)


@pytest.mark.parametrize("interval,position_index", [(2, 0), (63, 0), (64, 0), (65, 0), (127, 0), (129, 0), (17, 40), (64, 64)])
@pytest.mark.parametrize("q_heads,kv_heads", [(4, 4), (8, 1), (16, 2)])
def test_auto_never_picks_the_warp_level_kernel_from_16_packed_rows_up(interval, position_index, q_heads, kv_heads):
    """The shape sweep of the warp-level kernel's own test, left to the automatic choice: every chunk
    with at least 16 packed rows (rows x query heads per KV head) runs on the tensor-memory kernel."""
    case = Case(seed=200 + interval, interval=interval, batch=2, q_heads=q_heads, kv_heads=kv_heads,
                max_seq=position_index + interval + 5, position_index=position_index)
    want_k, want_v, want_o, want_l = case.oracle()
    got_k, got_v, got_o, got_l = case.gpu()
    assert_cache_bit_exact(got_k, got_v, want_k, want_v)
    assert_attention_close(case, got_o, got_l, want_o, want_l)
    name = "prefill_tcgen05" if interval * (q_heads // kv_heads) >= 16 else "prefill_warp_mma"
    assert case.last_stats[name][0] == 1


@pytest.mark.parametrize("interval,pos", [(40, 300), (300, 1000), (16, 127)])
def test_key_windows_that_start_past_key_zero(interval, pos):
    """Windows [0,a), [a,b), [b,inf) with a, b in the middle of 128-key tiles, on the tensor-memory
    kernel: their merged partials equal the unsplit result; rows that see no key of a window give
    an empty partial (O = 0, LSE = -inf)."""
    from helpers import from_bits
    dev = torch.device("cuda:0")
    case = Case(seed=70 + interval, interval=interval, batch=2, q_heads=8, kv_heads=2, max_seq=pos + interval,
                position_index=pos, poison=False)
    want_k, want_v, want_o, want_l = case.oracle()
    q = case.q.to(dev)
    ck = from_bits(want_k).view(2, 2, case.max_seq, 128).to(dev)
    cv = from_bits(want_v).view(2, 2, case.max_seq, 128).to(dev)
    out = torch.zeros_like(q)
    op = ellm_b200.Attention.new(q, ck, cv, out, 2, 8, 2, 128, case.strides, case.scale, max_seq=case.max_seq,
                                 max_interval=interval, prefill_kernel=L.PREFILL_TCGEN05)
    windows = [(0, 100), (100, pos + interval // 2), (pos + interval // 2, 1 << 40)]
    po = torch.full((len(windows), interval, 2, 8, 128), float("nan"), dtype=torch.float32, device=dev)
    pl = torch.full((len(windows), interval, 2, 8), float("nan"), dtype=torch.float32, device=dev)
    for i, (a, b) in enumerate(windows):
        op.run_window(pos, interval, 2, a, b, po[i], pl[i])
    assert op.kernel_stats()["prefill_tcgen05"][0] == len(windows)
    # rows before the last window's start see none of its keys
    empty = interval // 2
    assert (po[2, :empty] == 0).all() and (pl[2, :empty] == float("-inf")).all()
    rows = interval * 2 * 8
    lse = torch.zeros(rows, dtype=torch.float32, device=dev)
    ellm_b200.merge_partials(po.view(len(windows), rows, 128), pl.view(len(windows), rows), out, lse)
    torch.cuda.synchronize()
    assert_attention_close(case, bits(out), lse.view(interval, 2, 8).cpu().numpy(), want_o, want_l)


def test_more_items_than_sms_with_ragged_starts_and_with_the_fused_append():
    """The work list with several items per CTA in its two stateful corners: per-sequence chunk starts
    (the producer clears the tail of the last V tile of every item: a barrier whose phase carries from
    item to item) and the fused append (tiles waiting in ring slots to be stored into the cache while
    the next item's loads queue up).  5 sequences x 8 KV heads x 4 row-tile pairs = 160 items."""
    ragged = Case(seed=4321, interval=1024, batch=5, q_heads=8, kv_heads=8, max_seq=1700,
                  positions=[0, 300, 37, 512, 640], max_batch=6)
    _check(ragged)
    aligned = Case(seed=4322, interval=1024, batch=5, q_heads=8, kv_heads=8, max_seq=1300, position_index=256, max_batch=6)
    _check(aligned)          # starts on a key-tile boundary: the chunk's rows never pass through the append kernel
    assert aligned.last_stats["kv_append"][0] == 0
    shifted = Case(seed=4323, interval=1024, batch=5, q_heads=8, kv_heads=8, max_seq=1300, position_index=200, max_batch=6)
    _check(shifted)          # starts inside a key tile: the append kernel runs first
    assert shifted.last_stats["kv_append"][0] == 1


def test_one_cta_per_sm_and_one_cta_per_item_give_the_same_bits():
    """The work-item list walked by one CTA per SM (several items per CTA, barrier phases carried
    from item to item) against one CTA per item: 2 sequences x 4 KV heads x 24 row-tile pairs = 192
    items on 148 SMs, ragged steps per item."""
    dev = torch.device("cuda:0")
    S, B, Hq, Hkv = 768, 2, 32, 4
    g = torch.Generator().manual_seed(123)
    q = torch.randn(S, B, Hq, 128, generator=g).to(torch.bfloat16).to(dev)
    k = torch.randn(B, Hkv, S, 128, generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn(B, Hkv, S, 128, generator=g).to(torch.bfloat16).to(dev)
    outs = []
    for mode in (1, 0):
        out = torch.zeros_like(q)
        lse = torch.zeros(S, B, Hq, dtype=torch.float32, device=dev)
        op = ellm_b200.Attention.new(q, k, v, out, B, Hq, Hkv, 128, [Hkv * S * 128, S * 128, 128, 1], 0.088, max_seq=S,
                                     max_interval=S, lse=lse, prefill_kernel=L.PREFILL_TCGEN05)
        op.set_option("tc_persistent", mode)
        op.run(0, S, B, 1, 0)
        outs.append((out, lse))
        op.close()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert torch.isfinite(outs[0][0].float()).all()


def test_device_wait_timeout_on_an_enqueue_only_handle_shows_in_check():
    """A handle created with async = 1 only enqueues, so its run call cannot report a device-side
    wait that ran out; ellm_attn_check does, and clears the condition."""
    dev = torch.device("cuda:0")
    case = Case(seed=78, interval=256, batch=1, q_heads=1, kv_heads=1, max_seq=256, position_index=0, poison=False)
    _, _, want_o, want_l = case.oracle()
    q, ck, cv = case.q.to(dev), case.cache_k.to(dev), case.cache_v.to(dev)
    out = torch.zeros_like(q)
    lse = torch.zeros(256, 1, 1, dtype=torch.float32, device=dev)
    op = ellm_b200.Attention.new(q, ck, cv, out, 1, 1, 1, 128, case.strides, case.scale, max_seq=256, max_interval=256,
                                 lse=lse, k_new=case.k_new.to(dev), v_new=case.v_new.to(dev), prefill_kernel=L.PREFILL_TCGEN05,
                                 async_=True)
    op.check()                                           # nothing enqueued yet
    op.set_option("tc_wait_timeout_ns", 200_000_000)
    op.set_option("tc_debug_skip_kv_item", 0)            # the first K tile never arrives
    op.run(0, 256, 1, 1, 0)                              # returns at once, no error yet
    with pytest.raises(ellm_b200.EllmError) as e:
        op.check()
    assert e.value.status == L.ERR_DEVICE_TIMEOUT
    op.set_option("tc_debug_skip_kv_item", -1)
    op.run(0, 256, 1, 1, 0)
    op.check()                                           # cleared: the good run passes
    assert_attention_close(case, bits(out), lse.cpu().numpy(), want_o, want_l)
    op.close()


def test_device_wait_timeout_is_reported_and_the_context_stays_usable():
    """Failure detection without a fault: the kernel's loader is told to leave one K/V tile's
    barrier unsignalled (a flag that nothing sets), the wait on it runs out after the configured
    bound, the kernel releases tensor memory and returns, and the host call reports
    ELLM_ERR_DEVICE_TIMEOUT.  The same handle then runs normally and matches the oracle."""
    dev = torch.device("cuda:0")
    case = Case(seed=77, interval=256, batch=1, q_heads=1, kv_heads=1, max_seq=256, position_index=0)   # one CTA
    want_k, want_v, want_o, want_l = case.oracle()
    q, ck, cv = case.q.to(dev), case.cache_k.to(dev), case.cache_v.to(dev)
    out = torch.zeros_like(q)
    lse = torch.zeros(256, 1, 1, dtype=torch.float32, device=dev)
    op = ellm_b200.Attention.new(q, ck, cv, out, 1, 1, 1, 128, case.strides, case.scale, max_seq=256, max_interval=256,
                                 lse=lse, k_new=case.k_new.to(dev), v_new=case.v_new.to(dev), prefill_kernel=L.PREFILL_TCGEN05)
    op.set_option("tc_wait_timeout_ns", 200_000_000)     # 0.2 s
    op.set_option("tc_debug_skip_kv_item", 1)            # the first V tile never arrives
    with pytest.raises(ellm_b200.EllmError) as e:
        op.run(0, 256, 1, 1, 0)
    assert e.value.status == L.ERR_DEVICE_TIMEOUT
    op.set_option("tc_debug_skip_kv_item", -1)
    op.run(0, 256, 1, 1, 0)                              # same handle, same context
    assert_attention_close(case, bits(out), lse.cpu().numpy(), want_o, want_l)
    with pytest.raises(ellm_b200.EllmError):
        op.set_option("no_such_option", 1)


@pytest.mark.parametrize("boost", [6.0, 40.0, 300.0])
def test_scores_that_leap_above_the_running_maximum(boost):
    """Keys whose scores lie far above everything before them (mildly: within the range the fast path
    absorbs; strongly: tens of octaves, which must send the step down the rescaling path; and so far that
    the exponentials overflow before the rescale) - deep inside the sequence, in the middle of a key tile
    and at tile starts, so that steps after the first one meet them."""
    case = Case(seed=61, interval=1536, batch=1, q_heads=4, kv_heads=1, max_seq=1536, position_index=0)
    # columns 44, 45, 0, 0 of their key tiles (first half of a row: the step is redone from intact scores) and
    # columns 120, 64, 127 (second half: the first half's P has already gone to tensor memory and is rescaled there)
    for key in (300, 301, 640, 1024, 1400, 832, 1151):
        case.k_new[key] = (case.k_new[key].float() * boost).to(torch.bfloat16)
    want_k, want_v, want_o, want_l = case.oracle()
    got_k, got_v, got_o, got_l = case.gpu(prefill_kernel=L.PREFILL_TCGEN05)
    assert case.last_stats["prefill_tcgen05"][0] == 1
    assert_cache_bit_exact(got_k, got_v, want_k, want_v)
    assert_attention_close(case, got_o, got_l, want_o, want_l)
