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
"""
import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist

from . import Attention, merge_partials, sharding
from . import _lib as L


def _seeded_bf16(shape, seed, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    return torch.randn(shape, device=dev, generator=g).to(torch.bfloat16)


def _max_over_ranks(ms, dev, world):
    if world == 1:
        return ms
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _barrier(dev, world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)


def run_heads(args, rank, world, dev):
    """KV head hk of the full problem is generated from seed (base + hk) wherever it lives, so
    the result does not depend on the number of ranks."""
    S, Hq, Hkv, D = args.seq, args.q_heads, args.kv_heads, 128
    G = Hq // Hkv
    h0, h1 = sharding.kv_head_range(Hkv, world, rank)
    n = h1 - h0
    stream = torch.cuda.current_stream(dev).cuda_stream
    ms = 0.0
    out = lse = None
    if n > 0:
        q = torch.empty(S, 1, n * G, D, dtype=torch.bfloat16, device=dev)
        ck = torch.empty(1, n, S, D, dtype=torch.bfloat16, device=dev)
        cv = torch.empty_like(ck)
        for j, hk in enumerate(range(h0, h1)):
            q[:, 0, j * G:(j + 1) * G] = _seeded_bf16((S, G, D), args.seed * 1000 + 3 * hk, dev)
            ck[0, j] = _seeded_bf16((S, D), args.seed * 1000 + 3 * hk + 1, dev)
            cv[0, j] = _seeded_bf16((S, D), args.seed * 1000 + 3 * hk + 2, dev)
        out = torch.zeros_like(q)
        lse = torch.zeros(S, 1, n * G, dtype=torch.float32, device=dev)
        op = Attention.new(q, ck, cv, out, 1, n * G, n, D, [n * S * D, S * D, D, 1], 1.0 / np.sqrt(D), max_seq=S,
                           max_interval=S, lse=lse, device=dev.index, stream=stream, async_=True)
        for _ in range(args.warmup):
            op.run(0, S, 1, 1, 0)
    _barrier(dev, world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if n > 0:
        for _ in range(args.steps):
            op.run(0, S, 1, 1, 0)
    e1.record()
    _barrier(dev, world)
    ms = _max_over_ranks(e0.elapsed_time(e1) / args.steps, dev, world)
    if args.dump and n > 0:
        _dump_rows(args.dump, rank, q, ck, cv, out, lse, min(args.dump_rows, S))
    flops = 4 * D * Hq * S * (S + 1) / 2
    return {"mode": "heads", "ms": ms, "tflops": flops / ms / 1e9, "kv_heads_per_rank": n}


def _dump_rows(path, rank, q, ck, cv, out, lse, rows):
    """Saves the first `rows` rows of every local head (inputs and results) so that a test can
    compare them with a CPU checker; the first rows only need the first keys."""
    os.makedirs(path, exist_ok=True)
    torch.save({"q": q[:rows].cpu(), "k": ck[:, :, :rows].cpu(), "v": cv[:, :, :rows].cpu(),
                "out": out[:rows].cpu(), "lse": lse[:rows].cpu()}, os.path.join(path, f"rank{rank}.pt"))


def run_seq(args, rank, world, dev):
    S, Hq, Hkv, D = args.seq, args.q_heads, args.kv_heads, 128
    plan = sharding.SequenceChunkPlan(seq_len=S, world=world, zigzag=not args.contiguous)
    Lc = plan.chunk_len
    mine = plan.chunks_of(rank)
    stream = torch.cuda.current_stream(dev).cuda_stream
    scale = 1.0 / np.sqrt(D)
    # chunk c of the sequence is generated from seed (base + c) wherever it lives
    q_own = torch.stack([_seeded_bf16((Lc, 1, Hq, D), args.seed * 100000 + 3 * c, dev) for c in mine])
    kv = {c: (_seeded_bf16((1, Hkv, Lc, D), args.seed * 100000 + 3 * c + 1, dev),
              _seeded_bf16((1, Hkv, Lc, D), args.seed * 100000 + 3 * c + 2, dev)) for c in mine}
    strides = [Hkv * Lc * D, Lc * D, D, 1]
    q_all = torch.empty(world, len(mine), Lc, 1, Hq, D, dtype=torch.bfloat16, device=dev)
    q_buf = torch.empty(Lc, 1, Hq, D, dtype=torch.bfloat16, device=dev)
    dummy_out = torch.empty_like(q_buf)
    ops = {c: Attention.new(q_buf, kv[c][0], kv[c][1], dummy_out, 1, Hq, Hkv, D, strides, scale, max_seq=Lc,
                            max_interval=Lc, device=dev.index, stream=stream, async_=True) for c in mine}
    slot = {plan.chunks_of(r)[j]: (r, j) for r in range(world) for j in range(len(mine))}
    rows = Lc * Hq

    def compute_partial(i, k):
        r, j = slot[i]
        q_buf.copy_(q_all[r, j])
        o = torch.empty(Lc, 1, Hq, D, dtype=torch.float32, device=dev)
        lse = torch.empty(Lc, 1, Hq, dtype=torch.float32, device=dev)
        ops[k].run_window((i - k) * Lc, Lc, 1, 0, Lc, o, lse)
        return o, lse

    def merge(parts):
        o = torch.stack([p[0].view(rows, D) for p in parts])
        l = torch.stack([p[1].view(rows) for p in parts])
        mo = torch.empty(Lc, 1, Hq, D, dtype=torch.float32, device=dev)
        ml = torch.empty(Lc, 1, Hq, dtype=torch.float32, device=dev)
        merge_partials(o, l, mo, ml, device=dev.index, stream=stream, out_f32=True)
        return mo, ml

    use_p2p = args.exchange == "p2p" and world > 1
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

        def compute_partial_into(i, k, o, lse):
            r, j = slot[i]
            q_buf.copy_(q_all[r, j])
            if o is None:
                o = torch.empty(Lc, 1, Hq, D, dtype=torch.float32, device=dev)
                lse = torch.empty(Lc, 1, Hq, dtype=torch.float32, device=dev)
            ops[k].run_window((i - k) * Lc, Lc, 1, 0, Lc, o, lse)   # the kernel's stores go straight to o, local or peer
            return o, lse

        def merge_into(parts, o, lse):
            po = torch.stack([p[0].view(rows, D) for p in parts])
            pl = torch.stack([p[1].view(rows) for p in parts])
            merge_partials(po, pl, o, lse, device=dev.index, stream=stream, out_f32=True)

        def finish(i, n_sources):
            j = mine.index(i)
            mo = torch.empty(Lc, 1, Hq, D, dtype=torch.float32, device=dev)
            ml = torch.empty(Lc, 1, Hq, dtype=torch.float32, device=dev)
            merge_partials(views[rank][0][j, :n_sources].reshape(n_sources, rows, D),
                           views[rank][1][j, :n_sources].reshape(n_sources, rows), mo, ml, device=dev.index,
                           stream=stream, out_f32=True)
            return mo, ml

    def step():
        if world > 1:
            dist.all_gather_into_tensor(q_all.view(world, -1), q_own.view(-1))
        else:
            q_all[0].copy_(q_own)
        if use_p2p:
            return sharding.sequence_chunk_attention_p2p(plan, rank, compute_partial_into, merge_into, inbox_of,
                                                         lambda: hdl.barrier(channel=0), finish)
        return sharding.sequence_chunk_attention(plan, rank, None, compute_partial, merge, dist=dist,
                                                 empty_like=torch.empty_like)

    for _ in range(args.warmup):
        step()
    _barrier(dev, world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        result = step()
    e1.record()
    _barrier(dev, world)
    ms = _max_over_ranks(e0.elapsed_time(e1) / args.steps, dev, world)
    if args.dump:   # every owned chunk: all rows of q, k, v and of the merged result
        os.makedirs(args.dump, exist_ok=True)
        torch.save({c: {"q": q_own[mine.index(c)].cpu(), "k": kv[c][0].cpu(), "v": kv[c][1].cpu(),
                        "out": result[c][0].cpu(), "lse": result[c][1].cpu()} for c in mine},
                   os.path.join(args.dump, f"rank{rank}.pt"))
    flops = 4 * D * Hq * S * (S + 1) / 2
    pairs = [len(plan.pairs_of(r)) for r in range(world)]
    part_bytes = rows * D * 4 + rows * 4
    sent = sum(1 for i in range(plan.n_chunks) for src in plan.sources_of(i) if src != plan.owner(i))
    return {"mode": "seq", "ms": ms, "tflops": flops / ms / 1e9, "chunks": plan.n_chunks, "chunk_len": Lc,
            "zigzag": plan.zigzag, "pairs_per_rank": pairs, "exchange": "p2p" if use_p2p else "nccl", "nvlink_bytes_partials": sent * part_bytes,
            "nvlink_bytes_q_allgather": (world - 1) * world * q_own.numel() * 2}


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
    res = run_heads(args, rank, world, dev) if args.mode == "heads" else run_seq(args, rank, world, dev)
    res.update({"n_gpus": world, "seq": args.seq, "q_heads": args.q_heads, "kv_heads": args.kv_heads})
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
