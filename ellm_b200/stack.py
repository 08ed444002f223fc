"""Attention-only decoder stack: the callers either side of the attention operator.

Per layer, following the reference's decoder layer and attention block minus the MoE part
(src/qwen3_moe/decoder_layer.rs:139-165, src/qwen3_moe/attention.rs:126-196):

    h   = rms(x)                                   input norm, weight-free (generic/rms_norm.rs:6-26): ellm_rms_norm,
                                                   or inside MatMul3 (input_norm)
    q,k,v = h [Wq;Wk;Wv]^T                         matmul3 (src/compiler/mul/matmul3.rs:289-385), one GEMM
    q,k = rope(qk_norm(q, k)); cache <- k, v       ellm_qk_norm_rope_append
    a   = Attention(q, cache)                      ellm_attn_run
    x   = x + a Wo^T                               matmul_add (src/compiler/mul/matmul_add.rs:186-226)

With projections="tcgen05" (the default) every step runs on this repository's kernels
(ellm_b200/projection.py): MatMul3 and MatMulAdd pick the tcgen05 kernel with the norm + rope +
cache write (or the residual) in its epilogue for chunks, and the weight-streaming kernel for
decode steps of at most 16 rows.  projections="library" keeps torch / cuBLAS GEMMs followed by the
separate norm + rope + append kernel, as a comparison.  The input norm and attention are this
repository's kernels on both paths.  Decode steps can be captured once in a CUDA graph and
replayed: every kernel takes the per-sequence positions from a device array that the graph
itself advances.
"""
import numpy as np
import torch

from . import _lib as L
from .attention import Attention, qk_norm_rope_append, rms_norm
from .kv_cache import StaticKVCache
from .projection import MatMul3, MatMulAdd
from .rope import precompute_freqs_cis


class AttentionStack:
    def __init__(self, layers, hidden, q_heads, kv_heads, max_seq, max_interval, *, head_dim=128, theta=1e6,
                 eps=1e-6, seed=3, device="cuda:0", stream=None, max_batch=1, projections="tcgen05"):
        dev = torch.device(device)
        self.dev, self.layers, self.hidden = dev, layers, hidden
        self.q_heads, self.kv_heads, self.head_dim = q_heads, kv_heads, head_dim
        self.max_seq, self.max_interval, self.max_batch, self.eps = max_seq, max_interval, max_batch, eps
        self.stream = stream if stream is not None else torch.cuda.current_stream(dev)
        g = torch.Generator(device=dev).manual_seed(seed)

        def w(*shape, std=0.02, mean=0.0, dtype=torch.bfloat16):
            return (torch.randn(*shape, device=dev, generator=g) * std + mean).to(dtype)

        qd, kd = q_heads * head_dim, kv_heads * head_dim
        # N x K row-major, like the reference's W_nt (matmul3.rs:22-28); Wq, Wk, Wv are views of one
        # [Wq; Wk; Wv] matrix so that a decode step can stream them as one
        self.wqkv, self.wo = [], []
        for _ in range(layers):
            wq, wk, wv, wo = w(qd, hidden), w(kd, hidden), w(kd, hidden), w(hidden, qd)
            self.wqkv.append(torch.cat([wq, wk, wv]).contiguous())
            self.wo.append(wo)
        self.wq = [m[:qd] for m in self.wqkv]
        self.wk = [m[qd:qd + kd] for m in self.wqkv]
        self.wv = [m[qd + kd:] for m in self.wqkv]
        self.qkv = torch.zeros(max_interval * max_batch, qd + 2 * kd, dtype=torch.bfloat16, device=dev)
        self.h = torch.zeros(max_interval * max_batch, hidden, dtype=torch.bfloat16, device=dev)
        self.q_norm = [w(head_dim, mean=1.0, dtype=torch.float32) for _ in range(layers)]
        self.k_norm = [w(head_dim, mean=1.0, dtype=torch.float32) for _ in range(layers)]
        self.rope = torch.from_numpy(precompute_freqs_cis(head_dim, max_seq, theta)).to(dev)
        self.cache = StaticKVCache(layers, max_batch, kv_heads, max_seq, head_dim, device=dev)
        rows = max_interval * max_batch
        self.q = torch.zeros(max_interval, max_batch, q_heads, head_dim, dtype=torch.bfloat16, device=dev)
        self.a = torch.zeros_like(self.q)
        self.positions = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.scale = 1.0 / np.sqrt(head_dim)
        self.ops, self.qkv_ops, self.out_ops = [], [], []
        if projections not in ("tcgen05", "library"):
            raise ValueError("projections must be 'tcgen05' or 'library'")
        self.own_projections = projections == "tcgen05"
        self.x = torch.zeros(rows, hidden, dtype=torch.bfloat16, device=dev)   # the residual stream, updated in place
        dev_index, raw_stream = dev.index or 0, self.stream.cuda_stream
        for i in range(layers):
            ck, cv = self.cache.layer(i)
            self.ops.append(Attention.new(self.q, ck, cv, self.a, max_batch, q_heads, kv_heads, head_dim,
                                          self.cache.strides, self.scale, max_seq=max_seq, max_interval=max_interval,
                                          device=dev_index, stream=raw_stream, async_=True,
                                          # what precedes a decode step's attention here (the projection kernel, or the
                                          # norm + rope + append kernel) writes only Q and each sequence's newest cache row
                                          early_stream=True))
            if self.own_projections:
                # the layer's input norm rides inside the projection operator
                self.qkv_ops.append(MatMul3.new(self.x, self.wq[i], self.q, self.wk[i], ck, self.wv[i], cv, self.rope,
                                                head_dim, rows, hidden, qd, kd, kv_strides=self.cache.strides,
                                                max_batch=max_batch, max_seq=max_seq, rope_rows=max_seq, eps=eps,
                                                q_norm_weight=self.q_norm[i], k_norm_weight=self.k_norm[i],
                                                device=dev_index, stream=raw_stream, async_=True,
                                                input_norm_eps=eps, normed_scratch=self.h))
                self.out_ops.append(MatMulAdd.new(self.a, self.wo[i], self.x, self.x, rows, hidden, qd,
                                                  max_batch=max_batch, device=dev_index, stream=raw_stream, async_=True))
        self._rows = rows

    def _layer_tensor_core(self, i, n, batch, position_index, ragged):
        """One layer on self.x[:n * max_batch] in place, projections on this repository's kernels."""
        if ragged:
            self.qkv_ops[i].run_ragged(self.positions, n, batch)
            self.ops[i].run_ragged(self.positions, n, batch, 1, 0)
        else:
            self.qkv_ops[i].run(position_index, n, batch)
            self.ops[i].run(position_index, n, batch, 1, 0)
        self.out_ops[i].run(position_index, n, batch)

    def _layer(self, i, x, n, batch, position_index, ragged):
        """x: [n * max_batch, hidden] bf16 (rows ordered chunk row, then sequence)."""
        rows = n * self.max_batch
        dev_index = self.dev.index or 0
        h, qkv = self.h[:rows], self.qkv[:rows]
        rms_norm(x, h, self.eps, device=dev_index, stream=self.stream.cuda_stream)
        torch.matmul(h, self.wqkv[i].t(), out=qkv)
        q, a = self.q[:n], self.a[:n]
        qd, kd = self.q_heads * self.head_dim, self.kv_heads * self.head_dim
        ck, cv = self.cache.layer(i)
        # q, k, v are column blocks of the fused projection's output rows
        qk_norm_rope_append(qkv, qkv[:, qd:], qkv[:, qd + kd:], q, ck, cv, self.rope, self.cache.strides,
                            self.max_batch, self.q_heads, self.kv_heads, self.head_dim, self.max_seq, position_index,
                            n, batch, self.eps, q_weight=self.q_norm[i], k_weight=self.k_norm[i],
                            positions=self.positions if ragged else None, q_in_row_stride=qd + 2 * kd,
                            kv_in_row_stride=qd + 2 * kd, device=dev_index, stream=self.stream.cuda_stream)
        if ragged:
            self.ops[i].run_ragged(self.positions, n, batch, 1, 0)
        else:
            self.ops[i].run(position_index, n, batch, 1, 0)
        return torch.addmm(x, a.view(rows, -1), self.wo[i].t())

    def forward(self, x, position_index, batch=None, ragged=False):
        """One pass of all layers over a chunk: x [n, max_batch, hidden] -> same shape."""
        n = x.shape[0]
        batch = self.max_batch if batch is None else batch
        rows = n * self.max_batch
        y = x.reshape(rows, self.hidden)
        with torch.cuda.stream(self.stream):
            if self.own_projections:
                self.x[:rows].copy_(y)
                for i in range(self.layers):
                    self._layer_tensor_core(i, n, batch, position_index, ragged)
                y = self.x[:rows].clone()
            else:
                for i in range(self.layers):
                    y = self._layer(i, y, n, batch, position_index, ragged)
        return y.view(n, self.max_batch, self.hidden)

    def capture_decode_step(self, x_static):
        """Captures one decode step (all layers, positions read from self.positions and advanced
        by one at the end) into a CUDA graph; returns (graph, output tensor).  Replay with
        graph.replay() after writing the step's input into x_static."""
        # warm up outside the capture (library handles, cuBLAS workspaces)
        saved = self.positions.clone()
        for _ in range(2):
            self.forward(x_static, 0, ragged=True)
        self.stream.synchronize()
        self.positions.copy_(saved)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=self.stream):
            out = self.forward(x_static, 0, ragged=True)
            self.positions.add_(1)
        return graph, out

    def check(self):
        """Waits for the stream and raises if a bounded device-side wait of any operator's kernels
        ran out since the last check (the operators only enqueue)."""
        for op in self.ops + self.qkv_ops + self.out_ops:
            op.check()

    def close(self):
        for op in self.ops + self.qkv_ops + self.out_ops:
            op.close()
        self.cache.close()


def measure(layers=48, hidden=2048, q_heads=32, kv_heads=4, prefill=32768, decode=256, graph=True,
            projections="tcgen05", device="cuda:0"):
    """TTFT / TPOT of the attention path on the attention-only stack (BASELINE configs[3] by
    default): one timed prefill pass of `prefill` tokens over all layers after a warm-up pass, then
    `decode` single-token steps (a CUDA graph replayed per step unless graph=False).  Returns a dict."""
    dev = torch.device(device)
    torch.cuda.set_device(dev)
    stream = torch.cuda.Stream(dev)
    S = prefill
    max_seq = S + decode + 8
    stack = AttentionStack(layers, hidden, q_heads, kv_heads, max_seq, S, stream=stream, projections=projections,
                           device=device)
    g = torch.Generator(device=dev).manual_seed(3)
    x0 = torch.randn(S, 1, hidden, device=dev, generator=g).to(torch.bfloat16)
    with torch.cuda.stream(stream):
        stack.forward(x0, 0)            # warm-up pass (also fills the cache)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        y = stack.forward(x0, 0)
        e1.record(stream)
    stream.synchronize()
    stack.check()
    ttft = e0.elapsed_time(e1)
    flops_attn = 4 * 128 * q_heads * S * (S + 1) / 2 * layers
    flops_proj = 2 * S * hidden * (q_heads * 128 * 2 + kv_heads * 128 * 2) * layers
    # decode: positions start at S; the graph advances them
    x1 = y[-1:].clone()
    stack.positions.fill_(S)
    times = []
    with torch.cuda.stream(stream):
        if not graph:
            for _ in range(decode):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                x1 = stack.forward(x1, 0, ragged=True)
                stack.positions.add_(1)
                e1.record(stream)
                stream.synchronize()
                times.append(e0.elapsed_time(e1))
        else:
            cuda_graph, out = stack.capture_decode_step(x1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(decode):
                cuda_graph.replay()
                x1.copy_(out)
            e1.record(stream)
            stream.synchronize()
            times = [e0.elapsed_time(e1) / decode]
    stack.check()
    tpot = float(np.mean(times))
    kv_bytes = 2 * kv_heads * 128 * 2 * (S + decode / 2) * layers
    w_bytes = 2 * hidden * (q_heads * 128 * 2 + kv_heads * 128 * 2) * layers
    res = {
        "workload": f"{layers}-layer attention-only stack, hidden {hidden}, {q_heads} q / {kv_heads} kv heads, "
                    f"prefill {S} then {decode} decode steps, 1 sequence, synthetic weights and activations",
        "ttft_ms": ttft, "prefill_tflops": (flops_attn + flops_proj) / ttft / 1e9,
        "prefill_attention_flops_share": flops_attn / (flops_attn + flops_proj),
        "prefill_projections": projections, "tpot_ms": tpot, "decode_gbs": (kv_bytes + w_bytes) / tpot / 1e6,
        "decode_bytes_per_step": kv_bytes + w_bytes, "decode_cuda_graph": graph,
        "launches_per_decode_step": 4 * layers if projections == "tcgen05" else None,
        "final_positions": int(stack.positions[0]), "finite": bool(torch.isfinite(x1.float()).all())}
    stack.close()
    return res


def main():
    """python -m ellm_b200.stack --layers 48 --prefill 32768 --decode 256"""
    import argparse
    import json
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--q-heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--prefill", type=int, default=32768)
    ap.add_argument("--decode", type=int, default=256)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--projections", choices=["tcgen05", "library"], default="tcgen05")
    args = ap.parse_args()
    print(json.dumps(measure(args.layers, args.hidden, args.q_heads, args.kv_heads, args.prefill, args.decode,
                             not args.no_graph, args.projections)))


if __name__ == "__main__":
    main()
