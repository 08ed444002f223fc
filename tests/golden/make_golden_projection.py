"""Generates tests/golden/projection_golden.npz.

The reference's tests for its projection operators use all-ones operands only, and the reference
cannot be run where this repository builds (Rust nightly).  These vectors freeze the CPU oracle's
output for the whole step before attention - Q, K, V projections, per-head RMS norm, RoPE, cache
write - and for the output projection with residual, on small seeded non-uniform cases, after the
GEMM part of each case has been cross-checked against float64 numpy.  Run from the repository root:

    python tests/golden/make_golden_projection.py
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from helpers import bits  # noqa: E402

CASES = {
    # name: interval, max_batch, batch, q_heads, kv_heads, hidden, max_seq, position_index / positions
    "chunk_gqa": dict(seed=9101, interval=70, max_batch=2, batch=2, q_heads=4, kv_heads=2, hidden=192, max_seq=96, position_index=11),
    "decode_ragged": dict(seed=9102, interval=1, max_batch=4, batch=3, q_heads=8, kv_heads=2, hidden=256, max_seq=64,
                          positions=[0, 63, 17]),
}


def inputs(seed, interval, max_batch, batch, q_heads, kv_heads, hidden, max_seq, position_index=0, positions=None):
    g = torch.Generator().manual_seed(seed)
    m = interval * max_batch
    d = {
        "x": torch.randn(m, hidden, generator=g).to(torch.bfloat16),
        "wq": (torch.randn(q_heads * 128, hidden, generator=g) * 0.05).to(torch.bfloat16),
        "wk": (torch.randn(kv_heads * 128, hidden, generator=g) * 0.05).to(torch.bfloat16),
        "wv": (torch.randn(kv_heads * 128, hidden, generator=g) * 0.05).to(torch.bfloat16),
        "wo": (torch.randn(hidden, q_heads * 128, generator=g) * 0.05).to(torch.bfloat16),
        "qw": (1 + 0.02 * torch.randn(128, generator=g)).float(),
        "kw": (1 + 0.02 * torch.randn(128, generator=g)).float(),
    }
    return d


def run_oracle(kw):
    """Returns (q_out bits, K cache bits, V cache bits, output-projection bits); caches start at zero."""
    import ellm_b200
    d = inputs(**kw)
    interval, mb, batch = kw["interval"], kw["max_batch"], kw["batch"]
    hq, hkv, max_seq = kw["q_heads"], kw["kv_heads"], kw["max_seq"]
    rope = ellm_b200.precompute_freqs_cis(128, max_seq, 1e6)
    strides = [hkv * max_seq * 128, max_seq * 128, 128, 1]
    pq = oracle.matmul_nt_bf16(bits(d["x"]), bits(d["wq"]))
    ref = d["x"].float().numpy().astype(np.float64) @ d["wq"].float().numpy().astype(np.float64).T
    assert np.abs(oracle.bf16_bits_to_f32(pq) - ref).max() <= np.abs(ref).max() * 2.0 ** -8 + 1e-5   # float64 cross-check
    pk = oracle.matmul_nt_bf16(bits(d["x"]), bits(d["wk"]))
    pv = oracle.matmul_nt_bf16(bits(d["x"]), bits(d["wv"]))
    ck = np.zeros((mb, hkv, max_seq, 128), np.uint16)
    cv = np.zeros_like(ck)
    q = oracle.qk_norm_rope_append_bf16(pq.reshape(interval, mb, hq, 128), pk.reshape(interval, mb, hkv, 128),
                                        pv.reshape(interval, mb, hkv, 128), ck, cv, rope, strides, hq, hkv,
                                        kw.get("position_index", 0), interval, batch, 1e-6, q_weight=d["qw"].numpy(),
                                        k_weight=d["kw"].numpy(), positions=kw.get("positions"), max_batch=mb)
    y = oracle.matmul_nt_bf16(q.reshape(interval * mb, hq * 128), bits(d["wo"]), bits(d["x"]))
    return q, ck, cv, y


def main():
    blob = {}
    for name, kw in CASES.items():
        q, ck, cv, y = run_oracle(kw)
        blob[name + "/q"], blob[name + "/k_cache"], blob[name + "/v_cache"], blob[name + "/y"] = q, ck, cv, y
        blob[name + "/x_checksum"] = np.array([int(bits(inputs(**kw)["x"]).astype(np.uint64).sum())], dtype=np.uint64)
    path = os.path.join(HERE, "projection_golden.npz")
    np.savez_compressed(path, **blob)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
