"""Host-side sharding logic on CPU: partition rules, and the sequence-chunk exchange +
merge run as two gloo ranks with the CPU oracle standing in for the CUDA kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from ellm_b200 import sharding
from helpers import Case, bits


def test_assign_mirror_equals_the_oracle():
    for length in range(0, 40):
        for num in range(1, 9):
            for idx in range(num):
                assert sharding.assign(length, num, idx) == oracle.assign(length, num, idx)


def test_kv_head_ranges_cover_all_heads_once():
    for heads, world in ((8, 8), (8, 4), (8, 2), (4, 4), (4, 8), (5, 2)):
        got = [sharding.kv_head_range(heads, world, r) for r in range(world)]
        covered = [h for a, b in got for h in range(a, b)]
        assert covered == list(range(heads))


@pytest.mark.parametrize("zigzag", [False, True])
def test_sequence_chunk_plan_covers_the_causal_triangle_once(zigzag):
    for world in (1, 2, 4, 8):
        plan = sharding.SequenceChunkPlan(seq_len=64 * world, world=world, zigzag=zigzag)
        pairs = [p for r in range(world) for p in plan.pairs_of(r)]
        n = plan.n_chunks
        assert sorted(pairs) == sorted((i, k) for i in range(n) for k in range(i + 1))
        loads = [len(plan.pairs_of(r)) for r in range(world)]
        if zigzag:
            assert max(loads) == min(loads) == 2 * world + 1   # balanced
        else:
            assert loads == list(range(world, 0, -1))          # rank 0 does N pairs, the last does 1
        for c in range(n):
            assert c in plan.chunks_of(plan.owner(c))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, zigzag, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        S, Hq, Hkv = 64, 4, 2
        case = Case(seed=4242, interval=S, batch=1, q_heads=Hq, kv_heads=Hkv, max_seq=S, poison=False)
        plan = sharding.SequenceChunkPlan(seq_len=S, world=world, zigzag=zigzag)
        L = plan.chunk_len
        q = case.q.float().numpy()[:, 0]                       # [S, Hq, D]
        k = case.k_new.float().numpy()[:, 0]                   # [S, Hkv, D]
        v = case.v_new.float().numpy()[:, 0]
        g = Hq // Hkv

        def compute_partial(i, kc):                            # float64 softmax over key chunk kc
            o = np.zeros((L, Hq, 128), np.float32)
            lse = np.zeros((L, Hq), np.float32)
            for r in range(L):
                nkeys = L if kc < i else r + 1
                for h in range(Hq):
                    oo, ll = oracle.softmax_attention_f64(q[i * L + r, h], k[kc * L:kc * L + nkeys, h // g],
                                                          v[kc * L:kc * L + nkeys, h // g], case.scale)
                    o[r, h], lse[r, h] = oo, ll
            return torch.from_numpy(o), torch.from_numpy(lse)

        def merge(parts):
            o = np.stack([p[0].numpy().reshape(L * Hq, 128) for p in parts])
            l = np.stack([p[1].numpy().reshape(L * Hq) for p in parts])
            mo, ml = oracle.merge_partials(o, l)
            return torch.from_numpy(mo.reshape(L, Hq, 128)), torch.from_numpy(ml.reshape(L, Hq))

        got = sharding.sequence_chunk_attention(plan, rank, None, compute_partial, merge, dist=dist,
                                                empty_like=torch.empty_like)
        _, _, want_o, want_l = case.oracle(threads=1)
        want_o = oracle.bf16_bits_to_f32(want_o)[:, 0]
        worst_o = worst_l = 0.0
        for i, (o, lse) in got.items():
            worst_o = max(worst_o, float(np.abs(o.numpy() - want_o[i * L:(i + 1) * L]).max()))
            worst_l = max(worst_l, float(np.abs(lse.numpy() - want_l[i * L:(i + 1) * L, 0]).max()))
        ret[rank] = (sorted(got), worst_o, worst_l)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("zigzag", [False, True])
def test_sequence_chunk_exchange_two_gloo_ranks(zigzag):
    world, port = 2, _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(world, port, zigzag, ret), nprocs=world, join=True)
    plan = sharding.SequenceChunkPlan(seq_len=64, world=world, zigzag=zigzag)
    for rank in range(world):
        chunks, worst_o, worst_l = ret[rank]
        assert chunks == sorted(plan.chunks_of(rank))
        assert worst_o < 8e-3 and worst_l < 1e-4   # oracle O is bf16-rounded; merged partials are fp32


def _failing_rank_main(rank, world, port_a, port_b, ret):
    """Step 1: rank 1 leaves before its sends (it never enters the exchange); rank 0 must come
    back with ExchangeTimeout inside the bound instead of hanging.  Step 2: both ranks form a
    fresh group and the same exchange passes."""
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    plan = sharding.SequenceChunkPlan(seq_len=8, world=world, zigzag=True)
    L = plan.chunk_len

    def compute_partial(i, kc):   # the value of a partial is its (query chunk, key chunk) pair
        return torch.full((L, 128), float(10 * i + kc)), torch.zeros(L)

    def merge(parts):             # every partial starts with log-sum-exp 0, so the full merge is the mean
        mo, ml = oracle.merge_partials(np.stack([p[0].numpy() for p in parts]), np.stack([p[1].numpy() for p in parts]))
        return torch.from_numpy(mo), torch.from_numpy(ml)

    os.environ["MASTER_PORT"] = str(port_a)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    t0 = time.time()
    outcome = "left"
    if rank == 0:
        try:
            sharding.sequence_chunk_attention(plan, rank, None, compute_partial, merge, dist=dist,
                                              empty_like=torch.empty_like, timeout_s=2.0)
            outcome = "no error"
        except sharding.ExchangeTimeout:
            outcome = "timeout"
    elapsed = time.time() - t0
    # the survivor tells the host side (here: the rendezvous store) before anybody launches again
    store = dist.distributed_c10d._get_default_store()
    store.set(f"step1_rank{rank}", outcome)
    store.wait([f"step1_rank{r}" for r in range(world)], datetime.timedelta(seconds=30))
    dist.destroy_process_group()

    os.environ["MASTER_PORT"] = str(port_b)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        got = sharding.sequence_chunk_attention(plan, rank, None, compute_partial, merge, dist=dist,
                                                empty_like=torch.empty_like, timeout_s=20.0)
        ok = sorted(got) == sorted(plan.chunks_of(rank))
        for i, (o, _) in got.items():
            want = np.mean([10 * i + kc for kc in range(i + 1)])
            ok = ok and bool(torch.allclose(o, torch.full_like(o, float(want)), atol=1e-4))
        ret[rank] = (outcome, elapsed, ok)
    finally:
        dist.destroy_process_group()


def test_a_rank_that_leaves_before_its_sends_is_reported_within_the_bound():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_failing_rank_main, args=(world, _free_port(), _free_port(), ret), nprocs=world, join=True)
    outcome, elapsed, ok = ret[0]
    assert outcome == "timeout" and elapsed < 15.0
    assert ok and ret[1][2]      # the step on the fresh group gave the right result on both ranks
