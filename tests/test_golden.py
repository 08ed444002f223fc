"""The oracle against the committed golden vectors (CPU), and the CUDA path against the
same vectors (GPU).  tests/golden/make_golden.py generated them."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
from make_golden import CASES  # noqa: E402
from helpers import Case, assert_attention_close, bits  # noqa: E402

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention_golden.npz"))


def _rows(cache, case):
    c4 = cache.reshape(case.max_batch, case.kv_heads, case.max_seq, 128)
    return np.stack([c4[b, :, case.base(b):case.base(b) + case.interval] for b in range(case.batch)])


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_reproduces_golden(name):
    case = Case(**CASES[name])
    assert int(bits(case.q).astype(np.uint64).sum()) == int(GOLD[name + "/q_checksum"][0]), "seeded inputs changed"
    ck, cv, out, lse = case.oracle(threads=3)
    assert np.array_equal(out, GOLD[name + "/out"])
    assert np.array_equal(lse, GOLD[name + "/lse"])
    assert np.array_equal(_rows(ck, case), GOLD[name + "/k_rows"])
    assert np.array_equal(_rows(cv, case), GOLD[name + "/v_rows"])


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", [0, 1, 2])
@pytest.mark.parametrize("name", sorted(CASES))
def test_gpu_matches_golden(name, kernel):
    case = Case(**CASES[name])
    if kernel != 0 and case.interval == 1:
        pytest.skip("a decode step never reaches a prefill kernel; the choice of one changes nothing")
    gk, gv, go, gl = case.gpu(prefill_kernel=kernel)
    assert np.array_equal(_rows(gk, case), GOLD[name + "/k_rows"])   # bit-exact cache writes
    assert np.array_equal(_rows(gv, case), GOLD[name + "/v_rows"])
    assert_attention_close(case, go, gl, GOLD[name + "/out"], GOLD[name + "/lse"])
