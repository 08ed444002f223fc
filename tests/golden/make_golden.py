"""Generates tests/golden/attention_golden.npz.

The reference has no golden files for attention (its tests use uniform inputs only), and it
cannot be run where this repository builds (Rust nightly).  These vectors therefore freeze the
CPU oracle's output on small seeded non-uniform cases, after each case has been cross-checked
against an independent float64 two-pass softmax, so that a later change to the oracle or to the
input generator cannot go unnoticed.  Run from the repository root:

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from helpers import Case, bits  # noqa: E402

CASES = {
    # name: Case kwargs
    "decode_ragged_gqa": dict(seed=9001, interval=1, batch=3, q_heads=8, kv_heads=2, max_seq=140, positions=[4, 63, 129]),
    "decode_mha_uniform": dict(seed=9002, interval=1, batch=2, q_heads=4, kv_heads=4, max_seq=70, position_index=64),
    "prefill_chunk_gqa": dict(seed=9003, interval=65, batch=2, q_heads=4, kv_heads=2, max_seq=80, position_index=3, max_batch=3),
    "prefill_from_zero_mha": dict(seed=9004, interval=130, batch=1, q_heads=2, kv_heads=2, max_seq=130, position_index=0),
}


def float64_check(case, ck, cv, out, lse):
    kf = oracle.bf16_bits_to_f32(ck).reshape(case.max_batch, case.kv_heads, case.max_seq, 128)
    vf = oracle.bf16_bits_to_f32(cv).reshape(case.max_batch, case.kv_heads, case.max_seq, 128)
    qf = case.q.float().numpy()
    of = oracle.bf16_bits_to_f32(out)
    g = case.q_heads // case.kv_heads
    for h in range(case.interval):
        for b in range(case.batch):
            for qh in range(case.q_heads):
                n = case.base(b) + h + 1
                want, want_lse = oracle.softmax_attention_f64(qf[h, b, qh], kf[b, qh // g, :n], vf[b, qh // g, :n], case.scale)
                assert np.abs(of[h, b, qh] - want).max() < 8e-3
                assert abs(lse[h, b, qh] - want_lse) < 2e-5


def main():
    blob = {}
    for name, kw in CASES.items():
        case = Case(**kw)
        ck, cv, out, lse = case.oracle(threads=2)
        float64_check(case, ck, cv, out, lse)
        blob[name + "/out"] = out
        blob[name + "/lse"] = lse
        # the appended rows only (the rest of the cache is the seeded input)
        rows_k, rows_v = [], []
        for b in range(case.batch):
            base = case.base(b)
            rows_k.append(ck.reshape(case.max_batch, case.kv_heads, case.max_seq, 128)[b, :, base:base + case.interval])
            rows_v.append(cv.reshape(case.max_batch, case.kv_heads, case.max_seq, 128)[b, :, base:base + case.interval])
        blob[name + "/k_rows"] = np.stack(rows_k)
        blob[name + "/v_rows"] = np.stack(rows_v)
        blob[name + "/q_checksum"] = np.array([int(bits(case.q).astype(np.uint64).sum())], dtype=np.uint64)
    path = os.path.join(HERE, "attention_golden.npz")
    np.savez_compressed(path, **blob)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
