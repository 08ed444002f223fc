"""Multi-GPU drivers of the attention path: one process per GPU (torchrun), NCCL only where
the path has an exchange step.

  torchrun --nproc-per-node N -m ellm_b200.multi_gpu --mode heads --seq 131072 --q-heads 64 --kv-heads 8
  torchrun --nproc-per-node N -m ellm_b200.multi_gpu --mode seq   --seq 1048576 --q-heads 32 --kv-heads 4

`heads`: every rank owns a contiguous range of KV heads with their query heads and runs the
whole causal prefill for them; no collective.  `seq`: one sequence cut into chunks
(sharding.SequenceChunkPlan); partial (O, LSE) per key chunk, exchanged with NCCL
send/recv - or stored by the producing kernels straight into the owner's memory
(--exchange p2p) - and combined by the merge kernel.  Rank 0 prints one JSON line; times are CUDA
events, maximum over ranks.  `--dump DIR` saves inputs and results for an external check.

`heads_prefill` and `seq_prefill` are the same runs as functions (the benchmark calls them); given
sample positions they also hand back, on rank 0, the inputs and results of those query rows so
that a caller can recompute them with a CPU checker.
"""
import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist

from . import Attention, merge_partials_list, sharding

D = 128


def _seeded_bf16(shape, seed, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    return torch.randn(shape, device=dev, generator=g).to(torch.bfloat16)


def _max_over_ranks(values, dev, world):
    t = torch.tensor(values, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t.tolist()]


def _barrier(dev, world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)


def head_seeds(seed, hk):
    """Seeds of (Q, K, V) of KV head `hk` of the full problem: a head is generated from its own
    seeds wherever it lives, so the result does not depend on the number of ranks."""
    return seed * 1000 + 3 * hk, seed * 1000 + 3 * hk + 1, seed * 1000 + 3 * hk + 2


def chunk_seeds(seed, c):
    """Seeds of (Q, K, V) of sequence chunk `c`."""
    return seed * 100000 + 3 * c, seed * 100000 + 3 * c + 1, seed * 100000 + 3 * c + 2


def heads_prefill(S, Hq, Hkv, rank, world, dev, steps=3, warmup=1, seed=2, sample_positions=None, dump=None,
                  dump_rows=256):
    """Causal prefill of one sequence of S tokens, KV-head groups sharded over the ranks (strong
    scaling: the problem is fixed, a rank owns Hkv / world groups).  Returns (result, sample)."""
    G = Hq // Hkv
    h0, h1 = sharding.kv_head_range(Hkv, world, rank)
    n = h1 - h0
    stream = torch.cuda.current_stream(dev).cuda_stream
    op = None
    if n > 0:
        q = torch.empty(S, 1, n * G, D, dtype=torch.bfloat16, device=dev)
        ck = torch.empty(1, n, S, D, dtype=torch.bfloat16, device=dev)
        cv = torch.empty_like(ck)
        for j, hk in enumerate(range(h0, h1)):
            sq, sk, sv = head_seeds(seed, hk)
            q[:, 0, j * G:(j + 1) * G] = _seeded_bf16((S, G, D), sq, dev)
            ck[0, j] = _seeded_bf16((S, D), sk, dev)
            cv[0, j] = _seeded_bf16((S, D), sv, dev)
        out = torch.zeros_like(q)
        lse = torch.zeros(S, 1, n * G, dtype=torch.float32, device=dev)
        op = Attention.new(q, ck, cv, out, 1, n * G, n, D, [n * S * D, S * D, D, 1], 1.0 / np.sqrt(D), max_seq=S,
                           max_interval=S, lse=lse, device=dev.index, stream=stream, async_=True)
        for _ in range(warmup):
            op.run(0, S, 1, 1, 0)
    _barrier(dev, world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if n > 0:
        for _ in range(steps):
            op.run(0, S, 1, 1, 0)
    e1.record()
    _barrier(dev, world)
    if op is not None:
        op.check()   # the handle only enqueues: a device-side wait that ran out shows here
    ms = _max_over_ranks([e0.elapsed_time(e1) / steps], dev, world)[0]
    if dump and n > 0:
        _dump_rows(dump, rank, q, ck, cv, out, lse, min(dump_rows, S))
    sample = None
    if sample_positions is not None and rank == 0 and n > 0:
        # the rows of rank 0's first KV head, query heads in rotation
        rows = []
        for i, pos in enumerate(sample_positions):
            g = i % G
            rows.append({"pos": int(pos), "q_head": g, "q": q[pos, 0, g].float().cpu().numpy(),
                         "out": out[pos, 0, g].float().cpu().numpy(), "lse": float(lse[pos, 0, g])})
        sample = {"kv_head": h0, "k": ck[0, 0].float().cpu().numpy(), "v": cv[0, 0].float().cpu().numpy(), "rows": rows}
    flops = 4 * D * Hq * S * (S + 1) / 2
    if op is not None:
        op.close()
    return {"mode": "heads", "ms": ms, "tflops": flops / ms / 1e9, "kv_heads_per_rank": n, "collective": "none"}, sample


def _dump_rows(path, rank, q, ck, cv, out, lse, rows):
    """Saves the first `rows` rows of every local head (inputs and results) so that a test can
    compare them with a CPU checker; the first rows only need the first keys."""
    os.makedirs(path, exist_ok=True)
    torch.save({"q": q[:rows].cpu(), "k": ck[:, :, :rows].cpu(), "v": cv[:, :, :rows].cpu(),
                "out": out[:rows].cpu(), "lse": lse[:rows].cpu()}, os.path.join(path, f"rank{rank}.pt"))


def seq_prefill(S, Hq, Hkv, rank, world, dev, steps=1, warmup=1, seed=4, zigzag=True, exchange="nccl",
                sample_positions=None, sample_kv_head=0, dump=None, timeout_s=None):
    """Causal prefill of one sequence of S tokens cut into chunks over the ranks (strong scaling),
    one exchange step for the partial (O, LSE).  Returns (result, sample)."""
    plan = sharding.SequenceChunkPlan(seq_len=S, world=world, zigzag=zigzag)
    Lc = plan.chunk_len
    mine = plan.chunks_of(rank)
    stream = torch.cuda.current_stream(dev).cuda_stream
    scale = 1.0 / np.sqrt(D)
    # chunk c of the sequence is generated from its own seeds wherever it lives
    q_own = torch.stack([_seeded_bf16((Lc, 1, Hq, D), chunk_seeds(seed, c)[0], dev) for c in mine])
    kv = {c: (_seeded_bf16((1, Hkv, Lc, D), chunk_seeds(seed, c)[1], dev),
              _seeded_bf16((1, Hkv, Lc, D), chunk_seeds(seed, c)[2], dev)) for c in mine}
    strides = [Hkv * Lc * D, Lc * D, D, 1]
    # every rank's query chunks, gathered; a chunk pair reads its queries straight from here
    q_all = torch.empty(world, len(mine), Lc, 1, Hq, D, dtype=torch.bfloat16, device=dev) if world > 1 else q_own[None]
    dummy_out = torch.empty(Lc, 1, Hq, D, dtype=torch.bfloat16, device=dev)
    ops = {c: Attention.new(q_all[0, 0], kv[c][0], kv[c][1], dummy_out, 1, Hq, Hkv, D, strides, scale, max_seq=Lc,
                            max_interval=Lc, device=dev.index, stream=stream, async_=True) for c in mine}
    slot = {plan.chunks_of(r)[j]: (r, j) for r in range(world) for j in range(len(mine))}
    rows = Lc * Hq

    def new_partial():
        return (torch.empty(Lc, 1, Hq, D, dtype=torch.float32, device=dev),
                torch.empty(Lc, 1, Hq, dtype=torch.float32, device=dev))

    def compute_partial(i, k, o=None, lse=None):
        r, j = slot[i]
        if o is None:
            o, lse = new_partial()
        # the kernel's stores go straight to o / lse, which may be a peer's memory
        ops[k].run_window_q(q_all[r, j], (i - k) * Lc, Lc, 1, 0, Lc, o, lse)
        return o, lse

    def merge(parts, o=None, lse=None):
        if o is None:
            o, lse = new_partial()
        merge_partials_list([p[0] for p in parts], [p[1] for p in parts], o, lse, device=dev.index, stream=stream,
                            out_f32=True)
        return o, lse

    use_p2p = exchange == "p2p" and world > 1
    if use_p2p:
        # inbox in symmetric memory: [owned chunk slot, source rank, rows, D] fp32 and the LSEs behind it
        import torch.distributed._symmetric_memory as symm_mem
        n_own = len(mine)
        o_elems, l_elems = n_own * world * rows * D, n_own * world * rows
        inbox = symm_mem.empty(o_elems + l_elems, dtype=torch.float32, device=dev)
        hdl = symm_mem.rendezvous(inbox, dist.group.WORLD.group_name)
        views = {}
        for r in range(world):
            buf = hdl.get_buffer(r, (o_elems + l_elems,), torch.float32)
            views[r] = (buf[:o_elems].view(n_own, world, Lc, 1, Hq, D), buf[o_elems:].view(n_own, world, Lc, 1, Hq))

        def inbox_of(dst, i, src):
            j = plan.chunks_of(dst).index(i)
            return views[dst][0][j, src], views[dst][1][j, src]

        def finish(i, n_sources):
            j = mine.index(i)
            return merge([(views[rank][0][j, s], views[rank][1][j, s]) for s in range(n_sources)])

    marks = []

    def mark(name):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        marks.append((name, e))

    def step():
        del marks[:]
        mark("start")
        if world > 1:
            dist.all_gather_into_tensor(q_all.view(world, -1), q_own.view(-1))
        mark("q_gathered")
        if use_p2p:
            res = sharding.sequence_chunk_attention_p2p(plan, rank, compute_partial, merge, inbox_of,
                                                        lambda: hdl.barrier(channel=0), finish)
        else:
            res = sharding.sequence_chunk_attention(plan, rank, None, compute_partial, merge, dist=dist,
                                                    empty_like=torch.empty_like, mark=mark, timeout_s=timeout_s)
        mark("end")
        return res

    for _ in range(warmup):
        step()
    _barrier(dev, world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        result = step()
    e1.record()
    _barrier(dev, world)
    for op in ops.values():
        op.check()
    # phases of the last step on this rank: Q all-gather, local chunk pairs, exchange, final merge
    phase = {}
    for (a, ea), (b, eb) in zip(marks[:-1], marks[1:]):
        phase[b] = ea.elapsed_time(eb)
    names = ["q_gathered", "local_done", "exchanged", "end"]
    ms, *ph = _max_over_ranks([e0.elapsed_time(e1) / steps] + [phase.get(n, 0.0) for n in names], dev, world)
    if dump:   # every owned chunk: all rows of q, k, v and of the merged result
        os.makedirs(dump, exist_ok=True)
        torch.save({c: {"q": q_own[mine.index(c)].cpu(), "k": kv[c][0].cpu(), "v": kv[c][1].cpu(),
                        "out": result[c][0].cpu(), "lse": result[c][1].cpu()} for c in mine},
                   os.path.join(dump, f"rank{rank}.pt"))
    sample = None
    if sample_positions is not None and rank == 0:
        # K/V of one KV head over the whole sequence: the other ranks' chunks are regenerated here
        # from their seeds; the sampled rows must lie in chunks this rank owns
        k_full = np.empty((S, D), np.float32)
        v_full = np.empty((S, D), np.float32)
        for c in range(plan.n_chunks):
            if c in kv:
                kc, vc = kv[c]
            else:
                kc = _seeded_bf16((1, Hkv, Lc, D), chunk_seeds(seed, c)[1], dev)
                vc = _seeded_bf16((1, Hkv, Lc, D), chunk_seeds(seed, c)[2], dev)
            k_full[c * Lc:(c + 1) * Lc] = kc[0, sample_kv_head].float().cpu().numpy()
            v_full[c * Lc:(c + 1) * Lc] = vc[0, sample_kv_head].float().cpu().numpy()
            del kc, vc
        G = Hq // Hkv
        rows_out = []
        for n_, pos in enumerate(sample_positions):
            c, r = divmod(int(pos), Lc)
            if c not in mine:
                raise ValueError(f"sample position {pos} lies in chunk {c}, which rank 0 does not own")
            h = sample_kv_head * G + n_ % G
            o, l = result[c]
            rows_out.append({"pos": int(pos), "q_head": n_ % G, "q": q_own[mine.index(c)][r, 0, h].float().cpu().numpy(),
                             "out": o[r, 0, h].float().cpu().numpy(), "lse": float(l[r, 0, h])})
        sample = {"kv_head": sample_kv_head, "k": k_full, "v": v_full, "rows": rows_out}
    flops = 4 * D * Hq * S * (S + 1) / 2
    pairs = [len(plan.pairs_of(r)) for r in range(world)]
    part_bytes = rows * D * 4 + rows * 4
    sent = sum(1 for i in range(plan.n_chunks) for src in plan.sources_of(i) if src != plan.owner(i))
    for op in ops.values():
        op.close()
    return {"mode": "seq", "ms": ms, "tflops": flops / ms / 1e9, "chunks": plan.n_chunks, "chunk_len": Lc,
            "zigzag": plan.zigzag, "pairs_per_rank": pairs, "exchange": "p2p" if use_p2p else ("nccl" if world > 1 else "none"),
            "nvlink_bytes_partials": sent * part_bytes,
            "nvlink_bytes_q_allgather": (world - 1) * world * q_own.numel() * 2,
            "phase_ms_max_over_ranks": dict(zip(["q_allgather", "chunk_pairs", "partials_exchange", "final_merge"], ph)),
            "exchange_share": (ph[0] + ph[2]) / ms if ms > 0 else 0.0}, sample


def owned_sample_positions(S, world, n, zigzag=True, prefix=65536, seed=7):
    """`n` query positions inside the chunks rank 0 owns: three quarters in the first `prefix`
    tokens (only when that prefix lies inside rank 0's first chunk), the rest in its last chunk;
    chunk edges and 128-row tile edges are always included."""
    plan = sharding.SequenceChunkPlan(seq_len=S, world=world, zigzag=zigzag)
    Lc = plan.chunk_len
    mine = plan.chunks_of(0)
    rng = np.random.default_rng(seed)
    first_hi = min(prefix, Lc)
    base = [0, 1, 127, 128, 129, 255, 256, first_hi - 129, first_hi - 128, first_hi - 1]
    n_first = max(len(base), (3 * n) // 4) if len(mine) > 1 else n
    pos = base + [int(x) for x in rng.integers(0, first_hi, max(0, n_first - len(base)))]
    if len(mine) > 1:
        c0 = mine[-1] * Lc
        edge = [c0, c0 + 1, c0 + 127, c0 + 128, c0 + Lc - 129, c0 + Lc - 128, c0 + Lc - 1]
        pos += edge + [c0 + int(x) for x in rng.integers(0, Lc, max(0, n - len(pos) - len(edge)))]
    return pos[:max(n, len(base))] if len(mine) == 1 else pos


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=["heads", "seq"], required=True)
    ap.add_argument("--seq", type=int, required=True)
    ap.add_argument("--q-heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--seed", type=int, default=2)
    ap.add_argument("--dump", default="", help="directory: save inputs and results for an external check")
    ap.add_argument("--dump-rows", type=int, default=256, help="heads mode: rows per head to save")
    ap.add_argument("--contiguous", action="store_true", help="seq mode: rank r owns chunk r (no zig-zag)")
    ap.add_argument("--exchange", choices=["nccl", "p2p"], default="nccl",
                    help="seq mode: move the partials with NCCL send/recv, or let the producing kernels store them "
                         "directly into the owner's symmetric-memory inbox over NVLink")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.mode == "heads":
        res, _ = heads_prefill(args.seq, args.q_heads, args.kv_heads, rank, world, dev, args.steps, args.warmup, args.seed,
                               dump=args.dump or None, dump_rows=args.dump_rows)
    else:
        res, _ = seq_prefill(args.seq, args.q_heads, args.kv_heads, rank, world, dev, args.steps, args.warmup, args.seed,
                             zigzag=not args.contiguous, exchange=args.exchange, dump=args.dump or None)
    res.update({"n_gpus": world, "seq": args.seq, "q_heads": args.q_heads, "kv_heads": args.kv_heads})
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
