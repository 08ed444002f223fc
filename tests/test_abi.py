"""The C-ABI library loads and exports everything include/ellm_attn.h declares; the
argument checks that need no GPU behave.  CPU only: no compute call is made."""
import ctypes as C

import ellm_b200
from ellm_b200 import _lib as L


def test_library_exports_every_declared_symbol():
    lib = ellm_b200.load()
    names = ellm_b200.header_symbols()
    assert len(names) >= 14
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/ellm_attn.h but not exported"
    assert set(names) == set(L._SIGNATURES), "python binding and header disagree"
    assert lib.ellm_attn_abi_version() == 1


def test_product_library_carries_no_tuning_hooks():
    """The per-CTA time stamps of the decode chain and of the prefill kernel exist only in libraries built
    with -DELLM_CHAIN_TRACE / -DELLM_TC_TRACE (ellm_b200/chain_trace.py builds one beside the product)."""
    lib = ellm_b200.load()
    for name in ("ellm_debug_chain_trace", "ellm_debug_read_tc_trace"):
        assert not hasattr(lib, name)
    from ellm_b200 import chain_trace
    assert chain_trace.TRACE_LIB != ellm_b200.build.LIB and callable(chain_trace.build_trace_lib)


def test_status_strings():
    lib = ellm_b200.load()
    assert lib.ellm_status_string(0) == b"ok"
    assert lib.ellm_status_string(3) == b"device-side wait timed out"


def _desc(**kw):
    d = L.AttnDesc()
    d.q = d.k_cache = d.v_cache = d.out = 0x1000
    d.max_batch, d.q_heads, d.kv_heads, d.head_size = 1, 8, 2, 128
    d.kv_strides = (C.c_size_t * 4)(2 * 64 * 128, 64 * 128, 128, 1)
    d.max_seq, d.max_interval, d.scale = 64, 1, 0.088
    for k, v in kw.items():
        setattr(d, k, v)
    return d


def test_bad_descriptors_are_rejected_without_touching_a_gpu():
    lib = ellm_b200.load()
    h = C.c_void_p()
    cases = [
        (None, L.ERR_INVALID_ARG),
        (_desc(q=None), L.ERR_INVALID_ARG),
        (_desc(q_heads=7), L.ERR_INVALID_ARG),            # not a multiple of kv_heads
        (_desc(head_size=64), L.ERR_UNSUPPORTED),
        (_desc(k_cache=0x1004), L.ERR_INVALID_ARG),        # misaligned base
        (_desc(scale=0.0), L.ERR_INVALID_ARG),
        (_desc(k_new=0x2000), L.ERR_INVALID_ARG),          # k_new without v_new
        (_desc(dtype=3), L.ERR_UNSUPPORTED),
        (_desc(kv_strides=(C.c_size_t * 4)(100, 50, 4, 1)), L.ERR_INVALID_ARG),
        (_desc(kv_strides=(C.c_size_t * 4)(1024, 512, 128, 2)), L.ERR_UNSUPPORTED),
    ]
    for d, want in cases:
        rc = lib.ellm_attn_create(None if d is None else C.byref(d), C.byref(h))
        assert rc == want, (rc, want, lib.ellm_last_error())
        assert not h.value
        assert lib.ellm_last_error() != b""
    assert lib.ellm_attn_run(None, 0, 1, 1, 1, 0) == L.ERR_INVALID_ARG
    assert lib.ellm_attn_destroy(None) == L.OK


def test_standalone_entry_points_check_arguments():
    lib = ellm_b200.load()
    strides = (C.c_size_t * 4)(1024, 512, 128, 1)
    assert lib.ellm_kv_append(None, 0x1000, strides, 1, 1, 128, 8, 0, None, 1, 1, 0, None) == L.ERR_INVALID_ARG
    assert lib.ellm_kv_append(0x1000, 0x2000, strides, 1, 1, 128, 8, 8, None, 1, 1, 0, None) == L.ERR_INVALID_ARG  # past max_seq
    assert lib.ellm_kv_append(0x1000, 0x2000, strides, 1, 1, 64, 8, 0, None, 1, 1, 0, None) == L.ERR_UNSUPPORTED
    assert lib.ellm_attn_merge_partials(None, None, 1, 1, 128, None, None, 0, None) == L.ERR_INVALID_ARG
    assert lib.ellm_attn_merge_partials(0x1000, 0x1000, 0, 1, 128, 0x1000, None, 0, None) == L.ERR_INVALID_ARG
    out = C.c_void_p()
    assert lib.ellm_device_alloc(0, 0, C.byref(out)) == L.ERR_INVALID_ARG


def _desc3(**kw):
    d = L.MatMul3Desc()
    d.hidden = d.wq_nt = d.wk_nt = d.wv_nt = d.q_state = d.k_cache = d.v_cache = d.rope = 0x1000
    d.kv_strides = (C.c_size_t * 4)(2 * 64 * 128, 64 * 128, 128, 1)
    d.rope_rows, d.head_dim, d.m_row, d.col, d.b_q_row, d.b_kv_row = 64, 128, 16, 256, 1024, 256
    d.max_batch, d.max_seq, d.eps = 1, 64, 1e-6
    for k, v in kw.items():
        setattr(d, k, v)
    return d


def _desc_add(**kw):
    d = L.MatMulAddDesc()
    d.a = d.w_nt = d.output = 0x1000
    d.m_max, d.n_max, d.k_max, d.max_batch = 16, 256, 128, 1
    for k, v in kw.items():
        setattr(d, k, v)
    return d


def test_bad_projection_descriptors_are_rejected_without_touching_a_gpu():
    lib = ellm_b200.load()
    h = C.c_void_p()
    cases3 = [
        (None, L.ERR_INVALID_ARG),
        (_desc3(wk_nt=None), L.ERR_INVALID_ARG),
        (_desc3(head_dim=64), L.ERR_UNSUPPORTED),
        (_desc3(col=100), L.ERR_UNSUPPORTED),              # K not a multiple of 64
        (_desc3(b_q_row=1000), L.ERR_INVALID_ARG),         # not whole heads
        (_desc3(b_q_row=384), L.ERR_INVALID_ARG),          # 3 query heads over 2 KV heads
        (_desc3(m_row=15, max_batch=2), L.ERR_INVALID_ARG),
        (_desc3(hidden_row_stride=250), L.ERR_INVALID_ARG),
        (_desc3(hidden=0x1008), L.ERR_INVALID_ARG),        # misaligned base
        (_desc3(eps=-1.0), L.ERR_INVALID_ARG),
        (_desc3(input_norm=1), L.ERR_INVALID_ARG),         # input norm without a scratch
        (_desc3(kv_strides=(C.c_size_t * 4)(1024, 512, 128, 2)), L.ERR_UNSUPPORTED),
    ]
    for d, want in cases3:
        rc = lib.ellm_matmul3_create(None if d is None else C.byref(d), C.byref(h))
        assert rc == want, (rc, want, lib.ellm_last_error())
        assert not h.value
    cases_add = [
        (None, L.ERR_INVALID_ARG),
        (_desc_add(output=None), L.ERR_INVALID_ARG),
        (_desc_add(k_max=96), L.ERR_UNSUPPORTED),
        (_desc_add(n_max=100), L.ERR_UNSUPPORTED),
        (_desc_add(m_max=10, max_batch=4), L.ERR_INVALID_ARG),
        (_desc_add(a_row_stride=64), L.ERR_INVALID_ARG),   # shorter than a row
        (_desc_add(residual=0x1002), L.ERR_INVALID_ARG),
    ]
    for d, want in cases_add:
        rc = lib.ellm_matmul_add_create(None if d is None else C.byref(d), C.byref(h))
        assert rc == want, (rc, want, lib.ellm_last_error())
        assert not h.value
    assert lib.ellm_matmul3_run(None, 0, 1, 1, 1, 0) == L.ERR_INVALID_ARG
    assert lib.ellm_matmul_add_run(None, 0, 1, 1, 1, 0) == L.ERR_INVALID_ARG
    assert lib.ellm_matmul3_destroy(None) == L.OK and lib.ellm_matmul_add_destroy(None) == L.OK
    assert lib.ellm_matmul_check(None, 0) == L.ERR_INVALID_ARG
