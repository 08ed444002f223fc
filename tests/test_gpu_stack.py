"""The attention-only decoder stack (projections + norm/rope/append + attention + output
projection with residual) on a small configuration against a CPU restatement (B200 only).

The prefill chunk runs the projections on the tcgen05 kernel (fused epilogues), the decode steps on
the weight-streaming kernel (head norm, rotation and cache write inside); both sum in another order
than the CPU, so a projected value may land one bf16 step away
and the deviation grows a little through the layers; the tolerances here are for the whole stack,
the per-kernel parity bars are in the kernels' own tests."""
import numpy as np
import pytest
import torch

import ellm_b200
import oracle
from ellm_b200.stack import AttentionStack
from helpers import bits

pytestmark = pytest.mark.gpu


def _bf16(a):
    return oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(a.astype(np.float32)))


def _cpu_stack(stack, x, position_index, caches):
    """x [n, hidden] float32 holding bf16 values; caches: per layer (k bits, v bits)."""
    n = x.shape[0]
    Hq, Hkv, D = stack.q_heads, stack.kv_heads, 128
    rope = stack.rope.cpu().numpy()
    strides = stack.cache.strides
    for i in range(stack.layers):
        h = np.empty_like(x)
        for r in range(n):
            oracle.load().oracle_rms_norm_f32(x[r].ctypes.data, h[r].ctypes.data, x.shape[1], stack.eps)
        h = _bf16(h)
        q = _bf16(h @ stack.wq[i].float().cpu().numpy().T).reshape(n, 1, Hq, D)
        k = _bf16(h @ stack.wk[i].float().cpu().numpy().T).reshape(n, 1, Hkv, D)
        v = _bf16(h @ stack.wv[i].float().cpu().numpy().T).reshape(n, 1, Hkv, D)
        ck, cv = caches[i]
        qn = oracle.qk_norm_rope_append_bf16(oracle.f32_to_bf16_bits(q), oracle.f32_to_bf16_bits(k), oracle.f32_to_bf16_bits(v),
                                             ck, cv, rope, strides, Hq, Hkv, position_index, n, 1, stack.eps,
                                             q_weight=stack.q_norm[i].cpu().numpy(), k_weight=stack.k_norm[i].cpu().numpy())
        o, _ = oracle.attention_bf16(qn, ck, cv, strides, Hq, Hkv, stack.scale, position_index, n, 1)
        a = oracle.bf16_bits_to_f32(o).reshape(n, Hq * D)
        x = _bf16(x + a @ stack.wo[i].float().cpu().numpy().T)
    return x


def test_small_stack_prefill_then_decode_with_and_without_graph():
    dev = torch.device("cuda:0")
    layers, hidden, Hq, Hkv, S, steps = 3, 256, 4, 2, 150, 3
    stream = torch.cuda.Stream(dev)
    stack = AttentionStack(layers, hidden, Hq, Hkv, max_seq=S + steps + 4, max_interval=S, stream=stream, seed=11)
    g = torch.Generator().manual_seed(12)
    x0 = torch.randn(S, 1, hidden, generator=g).to(torch.bfloat16)
    y = stack.forward(x0.to(dev), 0)
    stream.synchronize()
    caches = [(np.zeros((1, Hkv, stack.max_seq, 128), np.uint16), np.zeros((1, Hkv, stack.max_seq, 128), np.uint16))
              for _ in range(layers)]
    want = _cpu_stack(stack, x0.float().numpy()[:, 0], 0, caches)
    got = y.float().cpu().numpy()[:, 0]
    d = np.abs(got - want)
    assert np.isfinite(got).all()
    assert d.mean() <= 1e-2 and d.max() <= 0.25, (d.mean(), d.max())
    # decode: eager step, then the same steps through a captured CUDA graph
    x1 = y[-1:].clone()
    stack.positions.fill_(S)
    eager = stack.forward(x1, 0, ragged=True).clone()
    stream.synchronize()
    want1 = _cpu_stack(stack, _bf16(got[-1:]), S, caches)
    d1 = np.abs(eager.float().cpu().numpy()[:, 0] - want1)
    assert d1.mean() <= 2e-2 and d1.max() <= 0.3, (d1.mean(), d1.max())
    graph, out = stack.capture_decode_step(x1)
    graph.replay()
    stream.synchronize()
    assert torch.equal(out, eager)             # same kernels, same inputs, same position
    assert int(stack.positions[0]) == S + 1    # the graph advanced the position itself
    for _ in range(steps - 1):
        x1.copy_(out)
        graph.replay()
    stream.synchronize()
    assert int(stack.positions[0]) == S + steps and torch.isfinite(out.float()).all()
    stack.close()


def test_tensor_core_and_library_projections_agree():
    dev = torch.device("cuda:0")
    layers, hidden, Hq, Hkv, S = 2, 512, 8, 2, 300
    outs, caches = [], []
    for mode in ("tcgen05", "library"):
        stream = torch.cuda.Stream(dev)
        stack = AttentionStack(layers, hidden, Hq, Hkv, max_seq=S + 4, max_interval=S, stream=stream, seed=21,
                               max_batch=2, projections=mode)
        g = torch.Generator().manual_seed(22)
        x0 = torch.randn(S, 2, hidden, generator=g).to(torch.bfloat16).to(dev)
        outs.append(stack.forward(x0, 0).float().cpu().numpy())
        stream.synchronize()
        caches.append([t.float().cpu().numpy() for t in stack.cache.layer(layers - 1)])
        if mode == "tcgen05":
            assert stack.qkv_ops[0].kernel_stats()[0] == 1 and stack.out_ops[0].kernel_stats()[0] == 1
        stack.close()
    d = np.abs(outs[0] - outs[1])
    assert np.isfinite(outs[0]).all() and d.mean() <= 5e-3 and d.max() <= 0.25, (d.mean(), d.max())
    for a, b in zip(caches[0], caches[1]):
        assert np.abs(a - b).mean() <= 2e-3
