"""Multi-GPU paths (needs >= 2 B200s in one box): KV-head-group sharding and sequence-chunk
sharding with the NCCL exchange of (O, LSE) partials, checked against the CPU oracle."""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

import oracle
from helpers import O_MAX_ABS, O_MEAN_ABS, LSE_MAX_ABS, bits

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(n, *args):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29631", "-m", "ellm_b200.multi_gpu", *args]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    return json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])


def _oracle_check(q, k, v, out, lse):
    """q [rows,1,Hq,D], k/v [1,Hkv,rows,D] (bf16 tensors), out bf16 or fp32, lse fp32."""
    rows, _, hq, _ = q.shape
    hkv = k.shape[1]
    want_o, want_l = oracle.attention_bf16(bits(q), bits(k), bits(v), [hkv * rows * 128, rows * 128, 128, 1], hq, hkv,
                                           1.0 / np.sqrt(128), 0, rows, 1, max_batch=1)
    d = np.abs(out.float().numpy() - oracle.bf16_bits_to_f32(want_o))
    assert d.max() <= O_MAX_ABS and d.mean() <= O_MEAN_ABS
    assert np.abs(lse.numpy() - want_l).max() <= LSE_MAX_ABS


def _need(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def test_head_group_sharding_two_gpus():
    _need(2)
    with tempfile.TemporaryDirectory() as d:
        res = _torchrun(2, "--mode", "heads", "--seq", "1024", "--q-heads", "16", "--kv-heads", "4", "--dump", d,
                        "--dump-rows", "300", "--steps", "1")
        assert res["n_gpus"] == 2 and res["kv_heads_per_rank"] == 2
        for r in range(2):
            t = torch.load(os.path.join(d, f"rank{r}.pt"))
            _oracle_check(t["q"], t["k"].contiguous(), t["v"].contiguous(), t["out"], t["lse"])


@pytest.mark.parametrize("layout,exchange", [("zigzag", "nccl"), ("contiguous", "nccl"), ("zigzag", "p2p"), ("contiguous", "p2p")])
def test_sequence_chunk_sharding_two_gpus(layout, exchange):
    _need(2)
    S, Hq, Hkv = 2048, 8, 2
    with tempfile.TemporaryDirectory() as d:
        extra = (["--contiguous"] if layout == "contiguous" else []) + ["--exchange", exchange]
        res = _torchrun(2, "--mode", "seq", "--seq", str(S), "--q-heads", str(Hq), "--kv-heads", str(Hkv), "--dump", d,
                        "--steps", "2", *extra)
        assert res["exchange"] == exchange
        chunks = {}
        for r in range(2):
            chunks.update(torch.load(os.path.join(d, f"rank{r}.pt")))
        n = res["chunks"]
        assert sorted(chunks) == list(range(n))
        q = torch.cat([chunks[c]["q"] for c in range(n)])                 # [S,1,Hq,D]
        k = torch.cat([chunks[c]["k"] for c in range(n)], dim=2)          # [1,Hkv,S,D]
        v = torch.cat([chunks[c]["v"] for c in range(n)], dim=2)
        out = torch.cat([chunks[c]["out"] for c in range(n)])
        lse = torch.cat([chunks[c]["lse"] for c in range(n)])
        _oracle_check(q, k.contiguous(), v.contiguous(), out, lse)
