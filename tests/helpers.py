"""Shared test helpers: seeded inputs, the oracle call, the GPU call, tolerances.

Parity bar of the attention path (bf16 in/out, fp32 accumulation):
  O   : max-abs <= 2e-2 and mean-abs <= 2e-3 against the oracle
  LSE : max-abs <= 1e-3 (fp32)
  KV-cache writes and indexing: bit-exact
"""
import numpy as np
import torch

import oracle

O_MAX_ABS = 2e-2
O_MEAN_ABS = 2e-3
LSE_MAX_ABS = 1e-3


def bits(t):
    """torch bf16 tensor -> numpy uint16 bit patterns (shares nothing with the GPU)."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def from_bits(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


def cache_strides(kv_heads, max_seq, head_dim=128):
    return [kv_heads * max_seq * head_dim, max_seq * head_dim, head_dim, 1]


class Case:
    """Seeded inputs of one operator step.

    Generation order per the benchmark's rule: Q, K, V from one torch generator,
    fp32 normal -> bf16.  `cache_k/v` hold the history (positions < base_b), and
    `k_new/v_new` the chunk's rows; rows past a sequence's end are poisoned with NaN
    so that any read of them shows up.
    """

    def __init__(self, seed, interval, batch, q_heads, kv_heads, max_seq, positions=None,
                 position_index=0, max_batch=None, head_dim=128, poison=True):
        g = torch.Generator().manual_seed(seed)
        self.interval, self.batch, self.q_heads, self.kv_heads = interval, batch, q_heads, kv_heads
        self.max_batch = max_batch or batch
        self.max_seq, self.head_dim = max_seq, head_dim
        self.positions = None if positions is None else np.asarray(positions, dtype=np.int32)
        self.position_index = position_index
        self.scale = 1.0 / np.sqrt(head_dim)
        mb = self.max_batch
        self.q = torch.randn(interval, mb, q_heads, head_dim, generator=g).to(torch.bfloat16)
        self.cache_k = torch.randn(mb, kv_heads, max_seq, head_dim, generator=g).to(torch.bfloat16)
        self.cache_v = torch.randn(mb, kv_heads, max_seq, head_dim, generator=g).to(torch.bfloat16)
        self.k_new = torch.randn(interval, mb, kv_heads, head_dim, generator=g).to(torch.bfloat16)
        self.v_new = torch.randn(interval, mb, kv_heads, head_dim, generator=g).to(torch.bfloat16)
        if poison:
            for b in range(mb):
                base = self.base(b) if b < batch else 0
                self.cache_k[b, :, base:, :] = float("nan")
                self.cache_v[b, :, base:, :] = float("nan")
        self.strides = cache_strides(kv_heads, max_seq, head_dim)

    def base(self, b):
        return int(self.positions[b]) if self.positions is not None else self.position_index

    def oracle(self, threads=0):
        """(cache_k bits after append, cache_v bits, out bits, lse) from the CPU oracle."""
        ck, cv = bits(self.cache_k).copy(), bits(self.cache_v).copy()
        for cache, new in ((ck, self.k_new), (cv, self.v_new)):
            oracle.kv_append_bf16(cache, bits(new), self.strides, self.max_batch, self.kv_heads,
                                  self.head_dim, self.position_index, self.interval, self.batch,
                                  positions=self.positions)
        out, lse = oracle.attention_bf16(bits(self.q), ck, cv, self.strides, self.q_heads,
                                         self.kv_heads, self.scale, self.position_index,
                                         self.interval, self.batch, max_batch=self.max_batch,
                                         positions=self.positions, threads=threads)
        return ck, cv, out, lse

    def gpu(self, prefill_kernel=0, use_run_host=False, cpu_num=1, device="cuda:0"):
        """Runs the CUDA path through the C ABI; returns the same tuple as oracle()."""
        from ellm_b200 import Attention
        dev = torch.device(device)
        q = self.q.to(dev)
        ck, cv = self.cache_k.to(dev), self.cache_v.to(dev)
        kn, vn = self.k_new.to(dev), self.v_new.to(dev)
        out = torch.full_like(q, float("nan"))
        lse = torch.full((self.interval, self.max_batch, self.q_heads), float("nan"),
                         dtype=torch.float32, device=dev)
        op = Attention.new(q, ck, cv, out, self.max_batch, self.q_heads, self.kv_heads,
                           self.head_dim, self.strides, self.scale, max_seq=self.max_seq,
                           max_interval=self.interval, lse=lse, k_new=kn, v_new=vn,
                           device=dev.index or 0, prefill_kernel=prefill_kernel)
        if use_run_host:
            qh = self.q.clone().pin_memory()
            oh = torch.zeros_like(qh).pin_memory()
            lh = torch.zeros(lse.shape, dtype=torch.float32).pin_memory()
            ph = None if self.positions is None else torch.from_numpy(self.positions)
            q.zero_()
            op.run_host(qh, oh, self.position_index, self.interval, self.batch,
                        k_new_host=self.k_new.contiguous(), v_new_host=self.v_new.contiguous(),
                        lse_host=lh, positions_host=ph)
            res_o, res_l = oh, lh
        elif self.positions is not None:
            pos = torch.from_numpy(self.positions).to(dev)
            for tid in range(cpu_num):
                op.run_ragged(pos, self.interval, self.batch, cpu_num, tid)
            res_o, res_l = out, lse
        else:
            # the reference's own test idiom: every thread id calls run
            for tid in range(cpu_num):
                op.run(self.position_index, self.interval, self.batch, cpu_num, tid)
            res_o, res_l = out, lse
        torch.cuda.synchronize(dev)
        self.last_stats = op.kernel_stats()
        op.close()
        return bits(ck), bits(cv), bits(res_o), res_l.detach().cpu().numpy()


def live_mask(case):
    """Boolean [interval, max_batch, q_heads] of rows the step actually computes."""
    m = np.zeros((case.interval, case.max_batch, case.q_heads), dtype=bool)
    m[:, :case.batch, :] = True
    return m


def assert_attention_close(case, got_out, got_lse, want_out, want_lse):
    m = live_mask(case)
    g = oracle.bf16_bits_to_f32(got_out)[m]
    w = oracle.bf16_bits_to_f32(want_out)[m]
    assert np.isfinite(g).all(), "non-finite output in a live row"
    diff = np.abs(g - w)
    assert diff.max() <= O_MAX_ABS, f"O max-abs {diff.max():.4g} > {O_MAX_ABS}"
    assert diff.mean() <= O_MEAN_ABS, f"O mean-abs {diff.mean():.4g} > {O_MEAN_ABS}"
    dl = np.abs(got_lse[m] - want_lse[m])
    assert dl.max() <= LSE_MAX_ABS, f"LSE max-abs {dl.max():.4g} > {LSE_MAX_ABS}"
    return diff.max(), diff.mean(), dl.max()


def assert_cache_bit_exact(got_k, got_v, want_k, want_v):
    assert np.array_equal(got_k, want_k), "K cache differs from the oracle's append"
    assert np.array_equal(got_v, want_v), "V cache differs from the oracle's append"
