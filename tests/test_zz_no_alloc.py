"""The allocation-free decode entry point against the handle-based one.

Some callers cannot allocate device memory while serving: everything was planned and
handed out when the graph was built, or another allocator in the process already owns
the GPU's memory.  For them `ellm_attn_decode_noalloc` keeps its split-KV partials in a
fixed array inside the library.  This file checks, through the C ABI, that it gives what
the existing entry point gives - on two calls in a row with different shapes, because the
array is shared and keeps the previous call's contents - and that it refuses sizes the
array cannot hold.  It is named to be collected last.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import ellm_b200
from ellm_b200 import _lib as L
from helpers import O_MAX_ABS, LSE_MAX_ABS, Case, bits

pytestmark = pytest.mark.gpu


def _both_ways(case, dev):
    """(out, lse) from the handle-based run_ragged and from decode_noalloc on the same cache."""
    pos = torch.from_numpy(case.positions).to(dev)
    q = case.q.to(dev)
    ck, cv = case.cache_k.to(dev), case.cache_v.to(dev)
    out_a = torch.full_like(q, float("nan"))
    lse_a = torch.full((1, case.max_batch, case.q_heads), float("nan"), dtype=torch.float32, device=dev)
    op = ellm_b200.Attention.new(q, ck, cv, out_a, case.max_batch, case.q_heads, case.kv_heads, 128, case.strides,
                                 case.scale, max_seq=case.max_seq, lse=lse_a, k_new=case.k_new.to(dev), v_new=case.v_new.to(dev))
    op.run_ragged(pos, 1, case.batch, 1, 0)   # appends the new rows, then attends
    op.close()
    out_b = torch.full_like(q, float("nan"))
    lse_b = torch.full_like(lse_a, float("nan"))
    ellm_b200.decode_noalloc(q, ck, cv, out_b, case.batch, case.q_heads, case.kv_heads, 128, case.strides, case.scale,
                             max_seq=case.max_seq, positions=pos, lse=lse_b)
    torch.cuda.synchronize(dev)
    return out_a, lse_a, out_b, lse_b


def test_noalloc_decode_matches_handle_decode_twice_in_a_row():
    dev = torch.device("cuda:0")
    # first call: long contexts, many pieces; second: fewer, shorter sequences and another
    # head layout, so stale partials from the first call would show if they were read
    cases = [
        Case(seed=301, interval=1, batch=6, q_heads=32, kv_heads=4, max_seq=4200, positions=[4100, 17, 2048, 999, 63, 3000]),
        Case(seed=302, interval=1, batch=2, max_batch=3, q_heads=8, kv_heads=8, max_seq=300, positions=[5, 257]),
    ]
    for case in cases:
        out_a, lse_a, out_b, lse_b = _both_ways(case, dev)
        live = slice(0, case.batch)
        a, b = out_a[:, live].float().cpu().numpy(), out_b[:, live].float().cpu().numpy()
        assert np.isfinite(b).all()
        assert np.abs(a - b).max() <= O_MAX_ABS
        assert np.abs(lse_a[:, live].cpu().numpy() - lse_b[:, live].cpu().numpy()).max() <= LSE_MAX_ABS
        # and against the CPU oracle, like every other parity test
        _, _, want_o, want_l = case.oracle()
        import oracle
        w = oracle.bf16_bits_to_f32(want_o)[:, live]
        assert np.abs(b - w).max() <= O_MAX_ABS
        assert np.abs(lse_b[:, live].cpu().numpy() - want_l[:, live]).max() <= LSE_MAX_ABS


def test_noalloc_decode_leaves_free_device_memory_unchanged():
    """What the entry point's name promises: once the first call on the device is behind it (that
    call is where the library image with its fixed array gets loaded), further calls take no
    device memory - free memory as the driver reports it is the same before and after."""
    dev = torch.device("cuda:0")
    case = Case(seed=303, interval=1, batch=4, q_heads=32, kv_heads=4, max_seq=1024, positions=[1000, 17, 512, 63])
    pos = torch.from_numpy(case.positions).to(dev)
    q, ck, cv = case.q.to(dev), case.cache_k.to(dev), case.cache_v.to(dev)
    ck[:, :, :1024] = torch.nan_to_num(ck[:, :, :1024])   # the rows at the positions themselves are read
    cv[:, :, :1024] = torch.nan_to_num(cv[:, :, :1024])
    out = torch.zeros_like(q)
    lse = torch.zeros(1, case.max_batch, case.q_heads, dtype=torch.float32, device=dev)

    def call():
        ellm_b200.decode_noalloc(q, ck, cv, out, case.batch, case.q_heads, case.kv_heads, 128, case.strides, case.scale,
                                 max_seq=case.max_seq, positions=pos, lse=lse)
    call()                                  # warm: symbol look-up, module load
    torch.cuda.synchronize(dev)
    free_before, _ = torch.cuda.mem_get_info(dev)
    for _ in range(8):
        call()
    torch.cuda.synchronize(dev)
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert free_after == free_before
    assert torch.isfinite(out[:, :case.batch].float()).all()


def test_noalloc_decode_rejects_sizes_beyond_its_scratch():
    dev = torch.device("cuda:0")
    lib = ellm_b200.load()
    buf = torch.zeros(4096, dtype=torch.bfloat16, device=dev)
    strides = (C.c_size_t * 4)(1024, 1024, 128, 1)
    p = buf.data_ptr()
    # 800 sequences * 1 kv head + 2 * SMs > 1024 slots
    rc = lib.ellm_attn_decode_noalloc(p, p, p, p, None, None, 0, 800, 1, 1, 128, strides, 8, 0.1, 0, None)
    assert rc == L.ERR_UNSUPPORTED and b"ELLM_NOALLOC_MAX_SLOTS" in lib.ellm_last_error()
    rc = lib.ellm_attn_decode_noalloc(p, p, p, p, None, None, 0, 2000, 1, 1, 128, strides, 8, 0.1, 0, None)
    assert rc == L.ERR_UNSUPPORTED and b"ELLM_NOALLOC_MAX_BATCH" in lib.ellm_last_error()
    rc = lib.ellm_attn_decode_noalloc(p, p, p, p, None, None, 0, 1, 1, 1, 64, strides, 8, 0.1, 0, None)
    assert rc == L.ERR_UNSUPPORTED
    torch.cuda.synchronize(dev)
