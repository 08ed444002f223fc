"""The oracle's projection path against the committed golden vectors (CPU), and the CUDA operators
against the same vectors (GPU).  tests/golden/make_golden_projection.py generated them."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
from make_golden_projection import CASES, inputs, run_oracle  # noqa: E402
from helpers import bits  # noqa: E402

import oracle  # noqa: E402

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "projection_golden.npz"))


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_reproduces_golden(name):
    kw = CASES[name]
    assert int(bits(inputs(**kw)["x"]).astype(np.uint64).sum()) == int(GOLD[name + "/x_checksum"][0]), "seeded inputs changed"
    q, ck, cv, y = run_oracle(kw)
    for got, key in ((q, "q"), (ck, "k_cache"), (cv, "v_cache"), (y, "y")):
        assert np.array_equal(got, GOLD[name + "/" + key]), key


def _near(got, want, exact_min, pair_steps):
    g32, w32 = oracle.bf16_bits_to_f32(got), oracle.bf16_bits_to_f32(want)
    assert np.isfinite(g32).all()
    assert (got == want).mean() >= exact_min, (got == want).mean()
    pair = np.abs(w32).reshape(-1, 2).max(axis=1, keepdims=True).repeat(2, axis=1).reshape(w32.shape)
    assert (np.abs(g32 - w32) <= pair_steps * pair * 2.0 ** -7 + 2e-4).all(), np.abs(g32 - w32).max()


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_gpu_matches_golden(name):
    import torch

    import ellm_b200
    kw = CASES[name]
    d = inputs(**kw)
    dev = "cuda:0"
    interval, mb, batch = kw["interval"], kw["max_batch"], kw["batch"]
    hq, hkv, hidden, max_seq = kw["q_heads"], kw["kv_heads"], kw["hidden"], kw["max_seq"]
    m = interval * mb
    strides = [hkv * max_seq * 128, max_seq * 128, 128, 1]
    rope = torch.from_numpy(ellm_b200.precompute_freqs_cis(128, max_seq, 1e6)).to(dev)
    ck = torch.zeros(mb, hkv, max_seq, 128, dtype=torch.bfloat16, device=dev)
    cv = torch.zeros_like(ck)
    q = torch.zeros(interval, mb, hq, 128, dtype=torch.bfloat16, device=dev)
    x = d["x"].to(dev)
    op = ellm_b200.MatMul3.new(x, d["wq"].to(dev), q, d["wk"].to(dev), ck, d["wv"].to(dev), cv, rope, 128, m, hidden, hq * 128,
                               hkv * 128, kv_strides=strides, max_batch=mb, max_seq=max_seq, rope_rows=max_seq,
                               q_norm_weight=d["qw"].to(dev), k_norm_weight=d["kw"].to(dev))
    if kw.get("positions") is not None:
        op.run_ragged(torch.tensor(kw["positions"], dtype=torch.int32, device=dev), interval, batch)
    else:
        op.run(kw.get("position_index", 0), interval, batch)
    _near(bits(q)[:, :batch], GOLD[name + "/q"][:, :batch], 0.97, 2)
    _near(bits(ck), GOLD[name + "/k_cache"], 0.97, 2)
    _near(bits(cv), GOLD[name + "/v_cache"], 0.99, 1)
    assert not bits(q)[:, batch:].any()   # dead sequence slots untouched
    # the output projection on the golden Q (so that the two operators are checked independently)
    from helpers import from_bits
    a = from_bits(GOLD[name + "/q"].reshape(m, hq * 128)).to(dev)
    y = x.clone()
    opa = ellm_b200.MatMulAdd.new(a, d["wo"].to(dev), y, y, m, hidden, hq * 128, max_batch=mb)
    opa.run(0, interval, batch)
    got = bits(y).reshape(interval, mb, hidden)
    _near(got[:, :batch], GOLD[name + "/y"].reshape(interval, mb, hidden)[:, :batch], 0.99, 1)
    assert np.array_equal(got[:, batch:], bits(d["x"]).reshape(interval, mb, hidden)[:, batch:])
    op.close()
    opa.close()
