"""Per-kernel timeline of one decode layer of the attention-only stack (a tuning tool; needs a B200).

Builds a second copy of the library with -DELLM_CHAIN_TRACE (ellm_b200/libellm_attn_trace.so: every CTA
of the decode-step kernels stores %globaltimer stamps at its start, after its griddepcontrol.wait, at one or
two points inside and at its end), runs the stack's captured decode step with it and prints, for two layers in
the middle of the stack, when the CTAs of each kernel started, passed their wait, finished their main loop and
ended.  The stamps cost about 2 us per layer; the product library carries none of this.

    python -m ellm_b200.chain_trace [--layers 12] [--context 32768]
"""
import argparse
import collections
import ctypes as C
import os
import shutil
import subprocess
import sys

import numpy as np

from . import build as _build

TRACE_LIB = os.path.join(_build.HERE, "libellm_attn_trace.so")
NAMES = {7: "QKV projection", 2: "decode", 3: "merge", 8: "output projection"}


def build_trace_lib():
    if os.path.exists(TRACE_LIB) and all(os.path.getmtime(src) <= os.path.getmtime(TRACE_LIB) for src in _build.sources()):
        return TRACE_LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc] + [f for f in _build.NVCC_FLAGS if f != "--use_fast_math=false"] + [
        "-DELLM_CHAIN_TRACE", "-I", _build.INCLUDE, "-o", TRACE_LIB, os.path.join(_build.CSRC, "ellm_attn_api.cu")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    return TRACE_LIB


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--context", type=int, default=32768)
    args = ap.parse_args()
    os.environ["ELLM_ATTN_LIB"] = build_trace_lib()    # before the package loads its library
    import torch
    import ellm_b200
    from .stack import AttentionStack

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = torch.cuda.Stream(dev)
    S, layers = args.context, args.layers
    stack = AttentionStack(layers, 2048, 32, 4, S + 64, S, stream=stream)
    g = torch.Generator(device=dev).manual_seed(3)
    x0 = torch.randn(S, 1, 2048, device=dev, generator=g).to(torch.bfloat16)
    with torch.cuda.stream(stream):
        y = stack.forward(x0, 0)
    stream.synchronize()
    x1 = y[-1:].clone()
    stack.positions.fill_(S)
    lib = ellm_b200.load()
    lib.ellm_debug_chain_trace.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
    with torch.cuda.stream(stream):
        graph, _ = stack.capture_decode_step(x1)
        for _ in range(6):
            graph.replay()
        stream.synchronize()
        if lib.ellm_debug_chain_trace(None, None, 1) != 0:
            raise RuntimeError("cannot reset the trace")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        graph.replay()
        e1.record(stream)
    stream.synchronize()
    print(f"decode step with stamps: {e0.elapsed_time(e1) * 1e3 / layers:.2f} us per layer ({layers} layers, context {S})")
    cap = 65536
    buf = np.zeros(cap * 6, dtype=np.uint64)
    n = C.c_uint(0)
    if lib.ellm_debug_chain_trace(buf.ctypes.data, C.byref(n), 0) != 0:
        raise RuntimeError("cannot read the trace")
    n = min(n.value, cap)
    r = buf[:n * 6].reshape(n, 6)
    kid = (r[:, 0] >> np.uint64(48)).astype(int)
    blk = (r[:, 0] & np.uint64(0xFFFFFFFF)).astype(int)
    t = r[:, 1:].astype(np.int64)        # start, waited, mid, mid2, end
    print("records:", dict(collections.Counter(kid)))
    launches = {}
    for k in NAMES:                       # one launch of kernel k per layer: split its records by start time
        idx = np.where(kid == k)[0]
        idx = idx[np.argsort(t[idx, 0], kind="stable")]
        per = len(idx) // layers if layers else 0
        launches[k] = [idx[i * per:(i + 1) * per] for i in range(layers)] if per else []

    def span(i, col, ref):
        v = t[i, col]
        v = v[v > 0]
        if len(v) == 0:
            return "      -      "
        return f"{(v.min() - ref) / 1e3:5.1f}..{(v.max() - ref) / 1e3:5.1f} (m {(np.median(v) - ref) / 1e3:5.1f})"

    for layer in (layers // 2, layers // 2 + 1):
        if layer >= layers or not launches[7]:
            continue
        ref = t[launches[7][layer], 0].min()
        print(f"--- layer {layer}: us after its QKV projection's first CTA started; first..last CTA (m = median)")
        print(f"{'kernel':18s} {'CTAs':>4s}  {'start':25s} {'wait returned':25s} {'mid':25s} {'mid2':25s} {'end':25s}")
        for k in (7, 2, 3, 8):
            if not launches[k]:
                continue
            i = launches[k][layer]
            print(f"{NAMES[k]:18s} {len(i):4d}  " + " ".join(f"{span(i, c, ref):25s}" for c in range(5)))
        i2 = launches[2][layer]
        last = i2[np.argsort(t[i2, 4])][-4:]
        print("   decode CTAs ending last: " + "; ".join(f"CTA {blk[j]} streamed by {(t[j, 2] - ref) / 1e3:.1f}, ended {(t[j, 4] - ref) / 1e3:.1f}" for j in last))
        if layer + 1 < layers:
            nxt = launches[7][layer + 1]
            w = t[nxt, 1]
            print(f"   next layer's QKV projection: first CTA at {(t[nxt, 0].min() - ref) / 1e3:.1f}, its wait returns at {(w[w > 0].min() - ref) / 1e3:.1f}")
    print("mid / mid2: projections - operands in shared memory / product loop done; decode - first piece streamed; merge - weighted sums done")
    stack.close()


if __name__ == "__main__":
    sys.exit(main())
