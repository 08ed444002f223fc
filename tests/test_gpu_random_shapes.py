"""Seeded sweep over shapes nobody picked by hand: batch, head counts, context lengths and chunk
starts drawn from a generator, every case checked against the CPU oracle through the C ABI.

The hand-written cases elsewhere sit on the tile edges (63/64/65, 127/128/129 ...); this file
covers the space between them.  Sizes are kept where the oracle finishes in seconds."""
import numpy as np
import pytest

from ellm_b200 import _lib as L
from helpers import Case, assert_attention_close, assert_cache_bit_exact

pytestmark = pytest.mark.gpu

_HEADS = [(1, 1), (2, 1), (4, 1), (8, 1), (16, 1), (4, 2), (8, 2), (6, 3), (8, 4), (12, 4), (32, 4), (16, 16), (24, 1)]
_TC_HEADS = [h for h in _HEADS if 128 % (h[0] // h[1]) == 0]   # the tensor-memory kernel wants a group dividing 128


def _check(case, **kw):
    want_k, want_v, want_o, want_l = case.oracle()
    got_k, got_v, got_o, got_l = case.gpu(**kw)
    assert_cache_bit_exact(got_k, got_v, want_k, want_v)
    assert_attention_close(case, got_o, got_l, want_o, want_l)


@pytest.mark.parametrize("seed", range(12))
def test_decode_step_drawn_shapes(seed):
    rng = np.random.default_rng(1000 + seed)
    q_heads, kv_heads = _HEADS[rng.integers(len(_HEADS))]
    batch = int(rng.integers(1, 9))
    max_batch = batch + int(rng.integers(0, 3))
    top = int(rng.choice([40, 300, 1500, 5000]))
    pos = [int(rng.integers(0, top)) for _ in range(batch)]
    case = Case(seed=seed, interval=1, batch=batch, max_batch=max_batch, q_heads=q_heads, kv_heads=kv_heads,
                max_seq=max(pos) + 1 + int(rng.integers(0, 70)), positions=pos)
    _check(case)
    assert case.last_stats["decode_splitkv"][0] == 1 and case.last_stats["merge"][0] == 1


@pytest.mark.parametrize("seed", range(8))
@pytest.mark.parametrize("kernel", [L.PREFILL_TCGEN05, L.PREFILL_WARP_MMA])
def test_prefill_chunk_drawn_shapes(seed, kernel):
    rng = np.random.default_rng(2000 + seed)
    heads = _TC_HEADS if kernel == L.PREFILL_TCGEN05 else _HEADS
    q_heads, kv_heads = heads[rng.integers(len(heads))]
    batch = int(rng.integers(1, 4))
    interval = int(rng.integers(2, 300))
    if rng.integers(2):
        # every sequence starts its chunk somewhere else
        pos = [int(rng.integers(0, 400)) for _ in range(batch)]
        case = Case(seed=50 + seed, interval=interval, batch=batch, q_heads=q_heads, kv_heads=kv_heads,
                    max_seq=max(pos) + interval + int(rng.integers(0, 70)), positions=pos)
    else:
        p0 = int(rng.integers(0, 400))
        case = Case(seed=50 + seed, interval=interval, batch=batch, q_heads=q_heads, kv_heads=kv_heads,
                    max_seq=p0 + interval + int(rng.integers(0, 70)), position_index=p0)
    _check(case, prefill_kernel=kernel)
    name = "prefill_tcgen05" if kernel == L.PREFILL_TCGEN05 else "prefill_warp_mma"
    assert case.last_stats[name][0] == 1
