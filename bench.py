#!/usr/bin/env python
"""Benchmark of the attention path: batched decode over the static KV cache.

Workload (N=1): 32 query / 4 KV heads, head_dim 128, bf16, 16 sequences with
context lengths uniform in [1024, 32768] (seed 1), cache [16, 4, 32768, 128] for K
and for V pre-filled N(0,1); one step = append one new token per sequence at
position len_b and attend over len_b + 1 keys (KV append, split-KV decode, merge).
The metric is the HBM rate of that step: algorithmic bytes / time, where the
algorithmic bytes are 2 (K,V) * kv_heads * 128 * 2 B * sum(len_b + 1) plus Q, O, LSE
and the appended rows.  Every step reads ~0.55 GB, far more than the 126 MB L2.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

With N > 1 (under torchrun) every rank runs the same workload on its own 16
sequences (independent sequences, no data-path collective): weak scaling of the
headline `value`.  The two shardings of ONE problem ride along in `extra.sharded`
at every N: the long causal prefill of BASELINE configs[2] split by KV-head group
(no collective) and, the 1M-token prefill of configs[4] split into zig-zag
sequence chunks with the NCCL exchange of (O, LSE) partials - strong scaling,
each with a parity stamp: sampled query rows recomputed by the CPU oracle on
rank 0, outside every timed region.  `--impl reference` times the CPU restatement
of the reference's AVX-512-FP16 attention kernel on all host cores instead (rank 0
only).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HQ, HKV, D, BATCH, MAX_SEQ = 32, 4, 128, 16, 32768
SCALE = 1.0 / np.sqrt(D)


def workload_lens():
    g = torch.Generator().manual_seed(1)
    return torch.randint(1024, 32769, (BATCH,), generator=g).to(torch.int32)


def algorithmic_bytes(lens):
    keys = int((lens.to(torch.int64) + 1).sum())
    kv = 2 * HKV * D * 2 * keys
    qo = 2 * BATCH * HQ * D * 2
    append = 2 * BATCH * HKV * D * 2
    lse = BATCH * HQ * 4
    return kv + qo + append + lse, kv + qo // 2  # (whole step, decode kernel alone: K/V + Q)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (no MEASURED_PEAKS.json)"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        # address the GPU by UUID: nvidia-smi's indices need not match CUDA's
        try:
            uuid = str(torch.cuda.get_device_properties(index).uuid)
            index = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:
            pass
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_reference_leg(lens, steps, warmup, budget_s=20.0):
    """The reference's CPU attention kernel (restated in oracle/) on all host cores, over the same
    16 sequences: the AVX-512-FP16 kernel where the host has avx512_fp16 (what the reference runs in
    production), else its generic fp32 kernel on a bounded sample of the sequences.
    Returns (GB/s, cores, sample text, ms per step, passes)."""
    import oracle
    from oracle.binding import aligned_empty
    lib = oracle.load()
    cores = os.cpu_count() or 1
    g = torch.Generator().manual_seed(1234)
    strides = [HKV * MAX_SEQ * D, MAX_SEQ * D, D, 1]
    have_f16 = bool(lib.oracle_f16_available())
    dt = torch.float16 if have_f16 else torch.bfloat16
    nseq = BATCH if have_f16 else 2          # the scalar fp32 kernel is ~50x slower: two sequences
    k = aligned_empty((BATCH, HKV, MAX_SEQ, D), np.uint16)
    v = aligned_empty((BATCH, HKV, MAX_SEQ, D), np.uint16)
    for b in range(nseq):  # only the rows a sequence reads need values
        n = int(lens[b]) + 1
        k[b, :, :n] = torch.randn(HKV, n, D, generator=g).to(dt).view(torch.int16).numpy().view(np.uint16)
        v[b, :, :n] = torch.randn(HKV, n, D, generator=g).to(dt).view(torch.int16).numpy().view(np.uint16)
    q = aligned_empty((1, BATCH, HQ, D), np.uint16)
    q[:] = torch.randn(1, BATCH, HQ, D, generator=g).to(dt).view(torch.int16).numpy().view(np.uint16)
    pos = lens.numpy().astype(np.int32)
    keys = int((lens[:nseq].to(torch.int64) + 1).sum())
    sample_bytes = 2 * HKV * D * 2 * keys + 2 * nseq * HQ * D * 2
    if have_f16:
        def once(reps):
            return oracle.attention_f16_timed(q, k, v, strides, HQ, HKV, SCALE, 0, 1, nseq, BATCH, positions=pos,
                                              threads=cores, repeats=reps)[1]
        kernel = "AVX-512-FP16 kernel"
    else:
        def once(reps):
            t0 = time.perf_counter()
            for _ in range(reps):
                oracle.attention_bf16(q, k, v, strides, HQ, HKV, SCALE, 0, 1, nseq, max_batch=BATCH, positions=pos,
                                      threads=cores)
            return time.perf_counter() - t0
        kernel = "generic fp32 kernel (host CPU lacks avx512_fp16)"
    for _ in range(max(1, warmup)):
        secs = once(1)
    reps = max(1, min(steps, int(budget_s / max(secs, 1e-3))))
    per = once(reps) / reps
    sample = (f"{'full workload' if nseq == BATCH else 'first %d of the' % nseq} 16 sequences, sum(len+1)={keys} keys, "
              f"32 query heads, {reps} passes, {kernel}, one pinned thread per core + spin barrier")
    return sample_bytes / per / 1e9, cores, sample, per * 1e3, reps


def cpu_info():
    model, flags = "", set()
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name") and not model:
                    model = line.split(":", 1)[1].strip()
                if line.startswith("flags") and not flags:
                    flags = set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return {"model": model, "avx512_fp16": "avx512_fp16" in flags, "amx_bf16": "amx_bf16" in flags,
            "amx_used": False}


def run_reference(args, lens):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    gbs, cores, sample, ms, reps = cpu_reference_leg(lens, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": "decode attn HBM GB/s", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": reps, "warmup": max(1, args.warmup), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16" if "FP16" in sample else "f32",
        "data": "synthetic", "config": config_dict(lens),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample, **cpu_info()},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "reference_scope": "one workload (16 sequences) on rank 0's host cores at every N; the GPU arm's value at N ranks "
                           "is the rate over N such workloads, so above N = 1 the ratio compares N GPUs with one host",
    }
    print(json.dumps(line))


def config_dict(lens):
    return {"workload": "batched decode attention over the static KV cache (BASELINE configs[1]): 16 sequences, "
                        "32 q / 4 kv heads, head_dim 128, bf16, context lengths U[1024,32768] seed 1, max_seq 32768",
            "batch": BATCH, "q_heads": HQ, "kv_heads": HKV, "head_dim": D, "max_seq": MAX_SEQ,
            "sum_len_plus_1": int((lens.to(torch.int64) + 1).sum()),
            "l2": "inputs larger than L2 (each step streams ~0.55 GB of K/V)",
            "per_rank": "every rank runs this workload on its own 16 sequences"}


def measured_tensor_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d["bf16_tflops_sustained"]), "measured (MEASURED_PEAKS.json)"
    return 1590.0, 1400.0, "fallback (no MEASURED_PEAKS.json)"


def prefill_long(dev, stream_ptr):
    """Secondary figure: the tcgen05 prefill kernel where it is not launch-bound - one sequence of
    32768 tokens, 32 q / 4 kv heads (one layer of BASELINE configs[3]); Q+K+V+O = 0.3 GB > L2."""
    from ellm_b200 import Attention
    S, Hq, Hkv = 32768, 32, 4
    g = torch.Generator(device=dev).manual_seed(3)
    q = torch.randn(S, 1, Hq, D, device=dev, generator=g).to(torch.bfloat16)
    ck = torch.randn(1, Hkv, S, D, device=dev, generator=g).to(torch.bfloat16)
    cv = torch.randn(1, Hkv, S, D, device=dev, generator=g).to(torch.bfloat16)
    out = torch.zeros_like(q)
    lse = torch.zeros(S, 1, Hq, dtype=torch.float32, device=dev)
    op = Attention.new(q, ck, cv, out, 1, Hq, Hkv, D, [Hkv * S * D, S * D, D, 1], SCALE, max_seq=S, max_interval=S,
                       lse=lse, device=dev.index, stream=stream_ptr, async_=True)
    for _ in range(3):
        op.run(0, S, 1, 1, 0)
    torch.cuda.synchronize(dev)
    times = []
    for _ in range(7):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); op.run(0, S, 1, 1, 0); e1.record()
        torch.cuda.synchronize(dev)
        times.append(e0.elapsed_time(e1))
    ms = statistics.median(times)
    flops = 4 * D * Hq * S * (S + 1) / 2
    burst, sustained, src = measured_tensor_peaks()
    tf = flops / ms / 1e9
    stats = op.kernel_stats()
    op.close()
    return {"workload": "causal prefill, seq 32768, 32 q / 4 kv heads, one layer (BASELINE configs[3] shape)",
            "kernel": "prefill_tcgen05_kernel" if stats["prefill_tcgen05"][0] else "prefill_warp_mma_kernel",
            "ms": ms, "tflops": tf,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": burst, "unit": "TFLOP/s", "frac": tf / burst,
                         "frac_of_sustained_peak": tf / sustained, "frac_of_nominal_2250": tf / 2250.0,
                         "peak_source": src + " bf16_tflops (burst: the kernel is timed alone)"}}


def projections_extra(dev, stream_ptr):
    """Secondary figures: the projections either side of attention at one layer of BASELINE
    configs[3] (hidden 2048, 32 q / 4 kv heads): the tcgen05 kernel on a 32768-row chunk, and the
    weight-streaming kernel on a one-row decode step (8 weight sets in rotation, 300 MB > L2)."""
    import ellm_b200
    from ellm_b200.projection import MatMul3, MatMulAdd
    S, hidden, Hq, Hkv = 32768, 2048, 32, 4
    qd, kd = Hq * D, Hkv * D
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(S, hidden, device=dev, generator=g).to(torch.bfloat16)
    wqkv = [(torch.randn(qd + 2 * kd, hidden, device=dev, generator=g) * 0.02).to(torch.bfloat16) for _ in range(8)]
    wo = [(torch.randn(hidden, qd, device=dev, generator=g) * 0.02).to(torch.bfloat16) for _ in range(8)]
    ck = torch.zeros(1, Hkv, S, D, dtype=torch.bfloat16, device=dev)
    cv = torch.zeros_like(ck)
    strides = [Hkv * S * D, S * D, D, 1]
    rope = torch.from_numpy(ellm_b200.precompute_freqs_cis(D, S, 1e6)).to(dev)
    q = torch.zeros(S, 1, Hq, D, dtype=torch.bfloat16, device=dev)
    a = torch.randn(S, qd, device=dev, generator=g).to(torch.bfloat16)
    y = torch.zeros(S, hidden, dtype=torch.bfloat16, device=dev)
    ones = torch.ones(D, device=dev)
    burst, sustained, src = measured_tensor_peaks()

    def timed(fn, reps, rounds=5):
        for _ in range(2):
            fn()
        torch.cuda.synchronize(dev)
        times = []
        for _ in range(rounds):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize(dev)
            times.append(e0.elapsed_time(e1) / reps)
        return statistics.median(times)

    out = {}
    qkv_ops = [MatMul3.new(x, w[:qd], q, w[qd:qd + kd], ck, w[qd + kd:], cv, rope, D, S, hidden, qd, kd, kv_strides=strides,
                           max_batch=1, max_seq=S, rope_rows=S, q_norm_weight=ones, k_norm_weight=ones, device=dev.index,
                           stream=stream_ptr, async_=True) for w in wqkv]
    out_ops = [MatMulAdd.new(a, w, y, y, S, hidden, qd, max_batch=1, device=dev.index, stream=stream_ptr, async_=True)
               for w in wo]
    ms = timed(lambda: qkv_ops[0].run(0, S, 1), 4)
    tf = 2.0 * S * hidden * (qd + 2 * kd) / ms / 1e9
    out["qkv_norm_rope_append_chunk"] = {"kernel": "proj_tcgen05_kernel", "rows": S, "ms": ms, "tflops": tf,
                                         "frac_of_measured_burst_peak": tf / burst}
    ms = timed(lambda: out_ops[0].run(0, S, 1), 4)
    tf = 2.0 * S * hidden * qd / ms / 1e9
    out["out_proj_residual_chunk"] = {"kernel": "proj_tcgen05_kernel", "rows": S, "ms": ms, "tflops": tf,
                                      "frac_of_measured_burst_peak": tf / burst}
    peak, peak_src = measured_peaks()

    def all_qkv():
        for op in qkv_ops:
            op.run(0, 1, 1)

    def all_out():
        for op in out_ops:
            op.run(0, 1, 1)

    ms = timed(all_qkv, 4) / len(qkv_ops)
    gbs = (qd + 2 * kd) * hidden * 2 / ms / 1e6
    out["qkv_decode_step"] = {"kernel": "proj_skinny_kernel (head norm, rotation and cache write inside)", "rows": 1, "us": ms * 1e3,
                              "weight_gbs": gbs, "frac_of_measured_hbm": gbs / peak}
    ms = timed(all_out, 4) / len(out_ops)
    gbs = hidden * qd * 2 / ms / 1e6
    out["out_proj_decode_step"] = {"kernel": "proj_skinny_kernel", "rows": 1, "us": ms * 1e3, "weight_gbs": gbs,
                                   "frac_of_measured_hbm": gbs / peak}
    out["peaks"] = {"bf16_tflops_burst": burst, "hbm_gbs": peak, "source": src}
    for op in qkv_ops + out_ops:
        op.close()
    return out


def prefill_extra(dev, stream_ptr, steps, warmup):
    """Secondary figure: causal prefill of BASELINE configs[0] (seq 2048, 32/32 heads)."""
    from ellm_b200 import Attention
    S, H = 2048, 32
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn(S, 1, H, D, device=dev, generator=g).to(torch.bfloat16)
    kn = torch.randn(S, 1, H, D, device=dev, generator=g).to(torch.bfloat16)
    vn = torch.randn(S, 1, H, D, device=dev, generator=g).to(torch.bfloat16)
    ck = torch.zeros(1, H, 4096, D, dtype=torch.bfloat16, device=dev)
    cv = torch.zeros_like(ck)
    out = torch.zeros_like(q)
    lse = torch.zeros(S, 1, H, dtype=torch.float32, device=dev)
    op = Attention.new(q, ck, cv, out, 1, H, H, D, [H * 4096 * D, 4096 * D, D, 1], SCALE, max_seq=4096,
                       max_interval=S, lse=lse, k_new=kn, v_new=vn, device=dev.index, stream=stream_ptr, async_=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    runs = 0
    for _ in range(max(3, warmup)):
        op.run(0, S, 1, 1, 0)
        runs += 1
    torch.cuda.synchronize(dev)
    times = []
    for _ in range(max(5, min(steps, 20))):
        runs += 1
        flush.zero_()  # write a buffer larger than L2 between timed iterations
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); op.run(0, S, 1, 1, 0); e1.record()
        torch.cuda.synchronize(dev)
        times.append(e0.elapsed_time(e1))
    ms = statistics.median(times)
    flops = 4 * D * H * S * (S + 1) / 2
    stats = op.kernel_stats()
    kernel = "prefill_tcgen05" if stats["prefill_tcgen05"][0] else "prefill_warp_mma"
    op.close()
    burst, sustained, src = measured_tensor_peaks()
    tf = flops / ms / 1e9
    return {"workload": "causal prefill, seq 2048, 32/32 heads (BASELINE configs[0]), KV append included, L2 flushed between iterations",
            "ttft_ms": ms, "tflops": tf, "kernel": kernel, "launches_per_step": sum(v[0] for v in stats.values()) // max(1, runs),
            "roofline": {"bound": "tensor", "achieved": tf, "peak": burst, "unit": "TFLOP/s", "frac": tf / burst,
                         "frac_of_nominal_2250": tf / 2250.0, "flops": flops,
                         "peak_source": src + " bf16_tflops (burst: the kernel is timed alone)"}}


def parity_stamp(sample, what):
    """Sampled query rows of a sharded run against the oracle's row kernel (the restatement of
    src/kernel/generic/flash_attention.rs:60-89) over all their keys; rank 0, outside any timed
    region.  `sample` comes from ellm_b200.multi_gpu (inputs and results of the rows)."""
    from concurrent.futures import ThreadPoolExecutor
    import oracle
    if sample is None:
        return None
    k, v = np.ascontiguousarray(sample["k"]), np.ascontiguousarray(sample["v"])

    def one(row):
        o = np.zeros(D, np.float32)
        want_l = oracle.flash_attention_f32(np.ascontiguousarray(row["q"], dtype=np.float32), k, v, o, float(SCALE), row["pos"])
        d = np.abs(row["out"] - o)
        return float(d.max()), float(d.mean()), abs(row["lse"] - want_l)

    with ThreadPoolExecutor(min(16, os.cpu_count() or 1)) as pool:
        res = list(pool.map(one, sample["rows"]))
    mx, mean, lse = max(r[0] for r in res), float(np.mean([r[1] for r in res])), max(r[2] for r in res)
    return {"rows": len(res), "max_abs": mx, "mean_abs": mean, "lse_max_abs": lse,
            "tolerance": {"max_abs": 2e-2, "mean_abs": 2e-3, "lse_max_abs": 1e-3},
            "ok": bool(mx <= 2e-2 and mean <= 2e-3 and lse <= 1e-3),
            "positions": [min(r["pos"] for r in sample["rows"]), max(r["pos"] for r in sample["rows"])],
            "checker": "CPU oracle row kernel (fp32 recurrence) over keys 0..=position, " + what}


def sharded_extra(rank, world, dev):
    """The two shardings of ONE problem (strong scaling), at this N."""
    from ellm_b200 import multi_gpu
    burst, sustained, src = measured_tensor_peaks()
    out = {}
    # (i) BASELINE configs[2]: seq 131072, 64 q / 8 kv heads, one KV-head group per GPU at N = 8
    S, Hq, Hkv = 131072, 64, 8
    n_rows = 64
    rng = np.random.default_rng(11)
    pos = [0, 1, 127, 128, 129, 255, 256, 4095, 4096, 65535, 65536, S - 129, S - 128, S - 2, S - 1]
    pos += [int(x) for x in rng.integers(0, S, n_rows - len(pos))]
    res, sample = multi_gpu.heads_prefill(S, Hq, Hkv, rank, world, dev, steps=2, warmup=1, seed=2, sample_positions=pos)
    if world > 1:
        # the same problem on rank 0's GPU alone, in the same run on the same box: what the N-rank time is compared with
        single = None
        if rank == 0:
            single, _ = multi_gpu.heads_prefill(S, Hq, Hkv, 0, 1, dev, steps=2, warmup=1, seed=2)
        torch.distributed.barrier()
        if rank == 0:
            res["single_gpu_ms_same_run"] = single["ms"]
            res["speedup_over_single_gpu"] = single["ms"] / res["ms"]
            res["strong_scaling_efficiency"] = single["ms"] / res["ms"] / min(world, Hkv)
        torch.cuda.empty_cache()
    if rank == 0:
        res["workload"] = ("BASELINE configs[2]: causal prefill, seq 131072, 64 q / 8 kv heads, KV-head groups sharded over the "
                           "ranks, no collective; strong scaling (fixed problem)")
        res["frac_of_n_x_sustained_peak"] = res["tflops"] / (min(world, Hkv) * sustained)
        res["parity"] = parity_stamp(sample, "rows of rank 0's first KV head, seed 2")
        out["head_groups"] = res
    del sample
    torch.cuda.empty_cache()
    # (ii) BASELINE configs[4]: seq 1048576, 32 q / 4 kv heads, zig-zag sequence chunks + partial exchange
    S, Hq, Hkv = 1048576, 32, 4
    pos = multi_gpu.owned_sample_positions(S, world, 64)
    res, sample = multi_gpu.seq_prefill(S, Hq, Hkv, rank, world, dev, steps=1, warmup=1 if world > 1 else 0, seed=4,
                                        sample_positions=pos)
    if world > 1:
        single = None
        if rank == 0:   # one GPU, the same code path (two chunks on one rank, no exchange), one step without warm-up
            single, _ = multi_gpu.seq_prefill(S, Hq, Hkv, 0, 1, dev, steps=1, warmup=0, seed=4)
        torch.distributed.barrier()
        if rank == 0:
            res["single_gpu_ms_same_run"] = single["ms"]
            res["speedup_over_single_gpu"] = single["ms"] / res["ms"]
            res["strong_scaling_efficiency"] = single["ms"] / res["ms"] / world
        torch.cuda.empty_cache()
    if rank == 0:
        res["workload"] = ("BASELINE configs[4]: causal prefill, seq 1048576, 32 q / 4 kv heads, 2N zig-zag sequence chunks; "
                           "Q all-gather + fp32 (O, LSE) partials over NCCL, merged by the owner; strong scaling"
                           + ("" if world > 1 else " (one rank: both chunks local, the window + merge path without the exchange; no warm-up step)"))
        res["frac_of_n_x_sustained_peak"] = res["tflops"] / (world * sustained)
        res["parity"] = parity_stamp(sample, "rows inside the 65536-token prefix and in rank 0's last chunk, seed 4")
        out["sequence_chunks"] = res
    del sample
    torch.cuda.empty_cache()
    if rank == 0:
        out["peaks"] = {"bf16_tflops_sustained": sustained, "bf16_tflops_burst": burst, "source": src}
    return out


def cpp_stack_decode():
    """The same decode step driven from compiled host code: tests/cpp/stack_decode_bench.cpp (the C++
    host mirror's asynchronous executor, one CUDA graph per step) built with g++ and run as a child
    process.  Returns its JSON line, or {"unavailable": why}."""
    import shutil
    import tempfile
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    gxx = shutil.which("g++")
    if not gxx:
        return {"unavailable": "no g++ on this box"}
    try:
        with tempfile.TemporaryDirectory() as tmp:
            exe = os.path.join(tmp, "stack_decode_bench")
            subprocess.run([gxx, "-std=c++17", "-O2", "-pthread", os.path.join(ROOT, "tests", "cpp", "stack_decode_bench.cpp"),
                            "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
                            "-L", os.path.join(ROOT, "ellm_b200"), "-lellm_attn", "-L", os.path.join(cuda, "lib64"), "-lcudart",
                            "-Wl,-rpath," + os.path.join(ROOT, "ellm_b200"), "-Wl,-rpath," + os.path.join(cuda, "lib64"), "-o", exe],
                           check=True, capture_output=True, text=True, timeout=300)
            res = subprocess.run([exe, "48", "32768", "256", "1"], capture_output=True, text=True, timeout=300)
            if res.returncode != 0:
                return {"unavailable": "stack_decode_bench failed: " + (res.stderr or res.stdout)[-300:]}
            return json.loads(res.stdout.strip().splitlines()[-1])
    except (subprocess.SubprocessError, OSError, ValueError) as e:
        return {"unavailable": f"{type(e).__name__}: {str(e)[-300:]}"}


def stack_extra(dev):
    """BASELINE configs[3]: 48-layer attention-only stack, 32768-token prefill then 256 decode steps."""
    from ellm_b200 import stack
    res = stack.measure(device=f"cuda:{dev.index}")
    torch.cuda.empty_cache()
    res["cpp_executor_decode"] = cpp_stack_decode()
    burst, sustained, src = measured_tensor_peaks()
    hbm, hsrc = measured_peaks()
    res["prefill_frac_of_sustained_peak"] = res["prefill_tflops"] / sustained
    res["prefill_frac_of_burst_peak"] = res["prefill_tflops"] / burst
    res["decode_frac_of_measured_hbm"] = res["decode_gbs"] / hbm
    res["peaks"] = {"bf16_tflops_sustained": sustained, "bf16_tflops_burst": burst, "hbm_gbs": hbm, "source": src}
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true")
    ap.add_argument("--no-sharded", action="store_true")
    ap.add_argument("--min-seconds", type=float, default=1.5, help="the timed rounds together last at least this long")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    lens = workload_lens()

    if args.impl == "reference":
        run_reference(args, lens)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention path has no CPU fallback")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    from ellm_b200 import Attention, StaticKVCache

    stream = torch.cuda.current_stream(dev)
    cache = StaticKVCache(1, BATCH, HKV, MAX_SEQ, D, device=dev)
    g = torch.Generator(device=dev).manual_seed(1 + 1000 * rank)
    for t in (cache.k, cache.v):
        for b in range(BATCH):
            t[0, b].copy_(torch.randn(HKV, MAX_SEQ, D, device=dev, generator=g))
    q = torch.randn(1, BATCH, HQ, D, device=dev, generator=g).to(torch.bfloat16)
    k_new = torch.randn(1, BATCH, HKV, D, device=dev, generator=g).to(torch.bfloat16)
    v_new = torch.randn(1, BATCH, HKV, D, device=dev, generator=g).to(torch.bfloat16)
    out = torch.zeros_like(q)
    lse = torch.zeros(1, BATCH, HQ, dtype=torch.float32, device=dev)
    positions = lens.to(dev)
    op = Attention.new(q, cache.k[0], cache.v[0], out, BATCH, HQ, HKV, D, cache.strides, SCALE,
                       max_seq=MAX_SEQ, max_interval=1, lse=lse, k_new=k_new, v_new=v_new,
                       device=local, stream=stream.cuda_stream, async_=True,
                       early_stream=True)   # the steps run back to back on resident inputs: nothing writes the positions
    total_bytes, kernel_bytes = algorithmic_bytes(lens)

    def step():
        op.run_ragged(positions, 1, BATCH, 1, 0)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, n):
        """n calls of fn between two events, a barrier and a synchronise on both sides; maximum over ranks."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def timed_rounds(fn, n, min_seconds, min_rounds, max_rounds=1000):
        """Rounds of exactly n steps each, until at least min_rounds rounds and min_seconds of timed work
        (the same count on every rank: it is fixed from the first round's maximum over ranks)."""
        first = timed(fn, n)
        rounds = int(min(max_rounds, max(min_rounds, np.ceil(min_seconds * 1e3 / max(first, 1e-3)))))
        return [first] + [timed(fn, n) for _ in range(rounds - 1)]

    for _ in range(args.warmup):
        step()
    op.check()
    before = op.kernel_stats()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
        warm_samples = len(sampler.rows)
    rounds = timed_rounds(step, args.steps, args.min_seconds, 25)
    if rank == 0:
        time.sleep(0.06)
        timed_samples = len(sampler.rows) - warm_samples
        sampler.rows = sampler.rows[warm_samples:]     # only what was sampled while the timed rounds ran
    after = op.kernel_stats()
    op.check()
    clocks = sampler.stop() if rank == 0 else None
    launches = sum(after[k][0] - before[k][0] for k in after) if rank == 0 else 0
    ms_per_step = statistics.median(rounds) / args.steps
    value = world * total_bytes / (ms_per_step * 1e-3) / 1e9

    # dominant kernel alone: CUDA events around each split-KV decode launch (a separate pass: the
    # events between the launches take away the overlap of a kernel's start with its predecessor's end)
    op.set_profiling(True)
    p0 = op.kernel_stats()["decode_splitkv"]
    for _ in range(5):
        timed(step, args.steps)
    p1 = op.kernel_stats()["decode_splitkv"]
    op.set_profiling(False)
    k_ms_serialized = (p1[2] - p0[2]) / max(1, p1[1] - p0[1])
    peak, peak_src = measured_peaks()
    # In the timed rounds the kernel's launches overlap their neighbours (dependent launches: a decode
    # grid moves in while the previous step's grid drains and its merge runs), so a launch has no
    # duration of its own there; what it takes of the stream's time is the step time - one launch per
    # step, the merge included, which makes the rate below a lower bound for the kernel.
    k_ms = ms_per_step
    achieved = kernel_bytes / (k_ms * 1e-3) / 1e9

    # end to end: host buffers in, host result out, through the host-buffer entry point
    qh = q.cpu().pin_memory(); knh = k_new.cpu().pin_memory(); vnh = v_new.cpu().pin_memory()
    oh = torch.zeros_like(qh).pin_memory()
    lh = torch.zeros(1, BATCH, HQ, dtype=torch.float32).pin_memory()
    ph = lens.clone().pin_memory()

    # the same host buffers every step (their contents are what a decode loop rewrites): arguments converted once
    step_host = op.bind_host(qh, oh, 0, 1, BATCH, k_new_host=knh, v_new_host=vnh, lse_host=lh, positions_host=ph)

    for _ in range(args.warmup):
        step_host()
    rounds_e2e = timed_rounds(step_host, args.steps, 0.5, 10)
    ms_e2e = statistics.median(rounds_e2e) / args.steps
    e2e = world * total_bytes / (ms_e2e * 1e-3) / 1e9
    h2d = qh.numel() * 2 + knh.numel() * 2 + vnh.numel() * 2 + ph.numel() * 4
    d2h = oh.numel() * 2 + lh.numel() * 4
    if not torch.isfinite(oh.float()).all():
        raise SystemExit("bench: non-finite attention output")
    op.close()
    del op, q, k_new, v_new, out, lse
    cache.close()
    torch.cuda.empty_cache()

    extra = {}
    if not args.no_extra and not args.no_sharded:
        extra["sharded"] = sharded_extra(rank, world, dev)

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    line = {
        "metric": "decode attn HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "rounds": {"count": len(rounds), "steps_per_round": args.steps, "ms_per_step_median": ms_per_step,
                   "ms_per_step_min": min(rounds) / args.steps, "ms_per_step_max": max(rounds) / args.steps,
                   "timed_ms_total": sum(rounds),
                   "how": "every round times exactly --steps steps between CUDA events with a barrier and a synchronise on "
                          "both sides, maximum over ranks; ms_per_step is the median round"},
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": config_dict(lens),
        "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e, "rounds": len(rounds_e2e), "entry": "ellm_attn_run_host",
                "transfer": "inside the timed call: one kernel fetches Q, new K/V rows and positions from the pinned host "
                            "buffers over PCIe, the merge kernel stores O and LSE into the pinned host buffers; no copy nodes"},
        "gpu_launches": launches,
        "clocks": dict(clocks, sampled="during the timed rounds only, every 50 ms", samples_in_timed_rounds=timed_samples),
        "roofline": {"bound": "hbm", "kernel": "decode_splitkv_kernel", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
                     "frac_of_nominal_8tbs": achieved / 8000.0, "kernel_ms": k_ms,
                     "kernel_ms_source": "the timed rounds themselves: CUDA events around --steps back-to-back steps, one launch of "
                                         "this kernel per step (its launches overlap their neighbours, so the step time - merge "
                                         "included - is what a launch takes of the stream: a lower bound on the kernel's rate)",
                     "serialized_kernel_ms": k_ms_serialized,
                     "serialized_frac": kernel_bytes / (k_ms_serialized * 1e-3) / 1e9 / peak,
                     "serialized_source": "separate pass of 5 rounds with CUDA events around every single launch of this kernel, "
                                          "which takes the overlap between launches away",
                     "algorithmic_bytes_per_launch": kernel_bytes, "traffic": TRAFFIC_BYTES_PER_LAUNCH,
                     "traffic_source": TRAFFIC_SOURCE},
        "tpot_attn_ms": ms_per_step,
    }
    if world == 1 and not args.no_cpu_baseline:
        leg = cpu_reference_leg(lens, 20, 1, budget_s=15.0)
        line["cpu_baseline"] = {"value": leg[0], "unit": "GB/s", "cores": leg[1], "kind": "port",
                                "sample": leg[2], "ms_per_step": leg[3], **cpu_info()}
    if world == 1 and not args.no_extra:
        extra["prefill"] = prefill_extra(dev, stream.cuda_stream, args.steps, args.warmup)
        extra["prefill_long"] = prefill_long(dev, stream.cuda_stream)
        extra["projections"] = projections_extra(dev, stream.cuda_stream)
        torch.cuda.empty_cache()
        extra["stack"] = stack_extra(dev)
    if extra:
        line["extra"] = extra
    print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one decode_splitkv_kernel launch on this workload
# (609.96 / 609.91 MB read + 4.51 / 4.61 MB written, two launches of decode_splitkv_kernel<1>), from an `ncu --set full --clock-control none
# -k regex:decode_splitkv -s 6 -c 2` capture of `python bench.py --steps 2 --warmup 3 --min-seconds 0.001
# --no-extra --no-cpu-baseline` on a B200.  A constant of that capture, not measured by this run.
TRAFFIC_BYTES_PER_LAUNCH = 614.49e6
TRAFFIC_SOURCE = "ncu capture of this workload (dram__bytes_read.sum + dram__bytes_write.sum, one launch); a recorded constant"

if __name__ == "__main__":
    main()
