"""Partitioning of the attention path over the GPUs of one node.

The reference has a single process and no communication layer (its only parallelism
is the thread split of src/compiler/assign.rs:11-38), so everything here is new
design; the split rule itself is the reference's `assign`.

Two ways to shard:

* KV-head groups (`kv_head_range`): rank r owns a contiguous range of KV heads with
  their query heads, and its slice of Q, cache and O lives only there.  Independent
  units: no data-path collective.  Sequences of a batch shard the same way.

* Sequence chunks of ONE long sequence (`SequenceChunkPlan`): the sequence is cut
  into chunks; each rank keeps the K/V rows of the chunks it owns and the matching
  query rows.  A query chunk i needs keys of every chunk k <= i, so the owner of k
  computes a partial (O, LSE) of Q_i against its K/V chunk k, the partials travel
  to the owner of i (one exchange step) and are combined there by the log-sum-exp
  merge.  With `zigzag` a rank owns chunks r and 2N-1-r, which evens out the causal
  triangle (every rank computes 2N+1 chunk pairs); contiguous ownership gives rank
  0 N pairs and rank N-1 one.

`sequence_chunk_attention` moves the partials with grouped send/recv (NCCL, or gloo in the CPU
tests).  `sequence_chunk_attention_p2p` needs no collective for them at all: every rank exposes
an inbox in symmetric memory and the kernel that produces a partial writes it straight into the
owner's inbox over NVLink (ordinary stores to a peer pointer), so the transfer rides in the
producing kernel's epilogue; one device-side barrier separates the writes from the merge.

The compute and merge steps are passed in as callables so that the same exchange
logic runs over NCCL with the CUDA kernels and, in the CPU tests, over gloo with a
stand-in.
"""
from dataclasses import dataclass


def assign(length, num, idx):
    """compiler::assign::assign: part `idx` of [0, length) split in `num` parts, the first
    length % num parts one longer; None when the part is empty."""
    if num <= 0 or not 0 <= idx < num:
        raise ValueError("idx must be in [0, num)")
    if length < idx + 1:
        return None
    q, r = divmod(length, num)
    if idx < r:
        b = (q + 1) * idx
        return b, b + q + 1
    b = q * idx + r
    return b, b + q


def kv_head_range(kv_heads, world, rank):
    """KV heads [h0, h1) owned by `rank`; its query heads are [h0*G, h1*G)."""
    part = assign(kv_heads, world, rank)
    return part if part else (0, 0)


@dataclass(frozen=True)
class SequenceChunkPlan:
    seq_len: int
    world: int
    zigzag: bool = True

    @property
    def n_chunks(self):
        return 2 * self.world if self.zigzag else self.world

    @property
    def chunk_len(self):
        if self.seq_len % self.n_chunks:
            raise ValueError(f"seq_len {self.seq_len} is not a multiple of {self.n_chunks} chunks")
        return self.seq_len // self.n_chunks

    def owner(self, chunk):
        if not self.zigzag:
            return chunk
        return chunk if chunk < self.world else 2 * self.world - 1 - chunk

    def chunks_of(self, rank):
        return [rank, 2 * self.world - 1 - rank] if self.zigzag else [rank]

    def pairs_of(self, rank):
        """(query chunk i, key chunk k) pairs `rank` computes: k owned by rank, i >= k."""
        return [(i, k) for k in self.chunks_of(rank) for i in range(k, self.n_chunks)]

    def sources_of(self, q_chunk):
        """Ranks that hold a partial for query chunk `q_chunk` (after their local pre-merge)."""
        return sorted({self.owner(k) for k in range(q_chunk + 1)})


def local_partials(plan, rank, compute_partial, merge):
    """Step 1 of the sharded prefill on `rank`: the partial of every (query chunk i, key chunk k)
    pair it computes, pre-merged per query chunk.  Returns {i: (o, lse)}."""
    local = {}
    for i, k in plan.pairs_of(rank):
        local.setdefault(i, []).append(compute_partial(i, k))
    return {i: (parts[0] if len(parts) == 1 else merge(parts)) for i, parts in local.items()}


def final_merge(plan, rank, local, received, merge):
    """Step 3: the owner combines its own partial of each owned query chunk with the ones it
    received ({i: [(o, lse), ...]}).  Returns {owned chunk index: (o, lse)}."""
    result = {}
    for i in plan.chunks_of(rank):
        parts = ([local[i]] if i in local else []) + list(received.get(i, []))
        result[i] = parts[0] if len(parts) == 1 else merge(parts)
    return result


class ExchangeTimeout(RuntimeError):
    """A peer did not deliver (or take) a partial within the bound: it has left or is stuck."""


def sequence_chunk_attention(plan, rank, q_chunks, compute_partial, merge, dist=None, empty_like=None, mark=None,
                             timeout_s=None):
    """Runs the sequence-chunk sharded prefill for `rank`.

    q_chunks: {chunk index: Q rows of that chunk} for EVERY chunk (the caller all-gathers Q
      first; with grouped-query attention Q is the larger operand but it is read-only).
    compute_partial(i, k) -> (o, lse): fp32 partial of query chunk i against key chunk k
      (k owned by this rank); k == i is causal inside the chunk, k < i sees the whole chunk.
    merge(list of (o, lse)) -> (o, lse): log-sum-exp combine (fp32 in, fp32 out).
    dist: torch.distributed (or None for world 1).  empty_like(o) allocates a receive buffer.
    mark(name): optional, called after the local chunk pairs ("local_done") and after the
      exchange ("exchanged") so that a caller can time the phases.
    timeout_s: bound of every wait of the exchange step.  A peer that left before its sends
      would otherwise block this rank for the process group's own timeout (minutes); with a bound
      the wait raises ExchangeTimeout and the caller can rebuild the group without that rank.
      None = wait as the backend does (on NCCL a wait only orders the stream).
    Returns {owned chunk index: (o, lse)} merged over all key chunks.
    """
    mark = mark or (lambda name: None)
    local = local_partials(plan, rank, compute_partial, merge)
    mark("local_done")

    # one exchange step: every partial goes to the owner of its query chunk
    mine = plan.chunks_of(rank)
    received = {i: [] for i in mine}
    ops = []
    if plan.world > 1:
        for i in range(plan.n_chunks):
            dst = plan.owner(i)
            for src in plan.sources_of(i):
                if src == dst:
                    continue
                if rank == src:
                    o, lse = local[i]
                    ops.append(dist.P2POp(dist.isend, o, dst))
                    ops.append(dist.P2POp(dist.isend, lse, dst))
                elif rank == dst:
                    ref_o, ref_l = next(iter(local.values()))
                    o, lse = empty_like(ref_o), empty_like(ref_l)
                    ops.append(dist.P2POp(dist.irecv, o, src))
                    ops.append(dist.P2POp(dist.irecv, lse, src))
                    received[i].append((o, lse))
        if ops:
            reqs = dist.batch_isend_irecv(ops)
            if timeout_s is None:
                for req in reqs:
                    req.wait()
            else:
                import datetime
                bound = datetime.timedelta(seconds=timeout_s)
                for req in reqs:
                    try:
                        done = req.wait(bound)
                    except RuntimeError as e:   # the backend's own text for a wait that ran out or a closed peer
                        raise ExchangeTimeout(f"rank {rank}: exchange of partials failed: {e}") from e
                    if done is False:
                        raise ExchangeTimeout(f"rank {rank}: a partial did not arrive within {timeout_s} s")
    mark("exchanged")
    return final_merge(plan, rank, local, received, merge)


def sequence_chunk_attention_p2p(plan, rank, compute_partial_into, merge_into, inbox_of, barrier, finish):
    """Sequence-chunk sharded prefill with the partials written directly into peer memory.

    inbox_of(dst_rank, q_chunk, src_rank) -> (o, lse): views of the fp32 inbox slot of `dst_rank`
      (its own memory when dst_rank == rank, a peer mapping otherwise) for the partial that
      `src_rank` contributes to query chunk `q_chunk`.
    compute_partial_into(i, k, o, lse): attention of query chunk i against key chunk k, result
      written to (o, lse) - which may be peer memory.
    merge_into(parts, o, lse): log-sum-exp combine of local partials into (o, lse).
    barrier(): device-side barrier over all ranks on the compute stream.
    finish(i, n_sources) -> result for owned chunk i from the first n_sources inbox slots.
    With zig-zag or contiguous ownership the ranks holding a partial for chunk i are always
    0 .. n_sources-1, so an owner's inbox slots for a chunk are contiguous.
    """
    barrier()   # nobody overwrites an inbox its owner may still be merging from the last step
    for i in range(plan.n_chunks):
        ks = [k for k in plan.chunks_of(rank) if k <= i]
        if not ks:
            continue
        o, lse = inbox_of(plan.owner(i), i, rank)
        if len(ks) == 1:
            compute_partial_into(i, ks[0], o, lse)
        else:
            merge_into([compute_partial_into(i, k, None, None) for k in ks], o, lse)
    barrier()   # every partial has landed in its owner's inbox
    result = {}
    for i in plan.chunks_of(rank):
        srcs = plan.sources_of(i)
        assert srcs == list(range(len(srcs)))
        result[i] = finish(i, len(srcs))
    return result
