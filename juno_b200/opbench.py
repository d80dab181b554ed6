"""Single-operator timings on device-resident data: the fused dequant-GEMV sweep and the attention sweep.

    python -m juno_b200.opbench gemv [--types q4_k,q6_k,q8_0] [--shapes 4096x4096,...] [--batches 1,4,16,64]
    python -m juno_b200.opbench attn [--ctx 512,2048,8192,32768] [--batches 1,8,64]

Weights are rotated over enough copies to exceed the 126 MB L2, x and y stay in HBM, and each launch is
timed with CUDA events on the context stream.  Prints one JSON line per case (GB/s = algorithmic bytes / time).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

import numpy as np

from . import _lib, synth
from ._lib import check
from .matvec import B200MatVec, GpuContext, PagedKvCache, _ptr

TYPES = {"q4_k": synth.Q4_K, "q6_k": synth.Q6_K, "q8_0": synth.Q8_0}
BPW = {synth.Q4_K: 144 / 256, synth.Q6_K: 210 / 256, synth.Q8_0: 34 / 32}
L2_BYTES = 126e6


def gemv_case(ctx, mv, t, rows, cols, batch, iters, warmup, seed=1, chain=0):
    import torch
    rng = np.random.default_rng(seed)
    wbytes = rows * cols * BPW[t]
    copies = max(1, min(24, int(np.ceil(2 * L2_BYTES / wbytes))))
    raw = synth.random_blocks(rng, t, rows, cols)
    mats = [mv.upload_quantized(raw, t, rows, cols) for _ in range(copies)]
    x = torch.from_numpy(rng.standard_normal((batch, cols)).astype(np.float32)).cuda()
    y = torch.empty((batch, rows), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    stream = torch.cuda.ExternalStream(ctx.stream())
    L = ctx._L

    def launch(i):
        check(L.juno_gemv_device(ctx.handle, mats[i % copies].handle, C.c_void_p(x.data_ptr()), batch,
                                 C.c_void_p(y.data_ptr()), None), "juno_gemv_device")

    for i in range(warmup):
        launch(i)
    name = [k for k, v in TYPES.items() if v == t][0]
    algo = wbytes + batch * cols * 4 + batch * rows * 4
    if chain:
        # `chain` launches back to back inside one CUDA graph: the per-launch time a product costs inside a decode step
        # (launch latency overlapped by programmatic dependent launch), not the time of an isolated launch
        g = torch.cuda.CUDAGraph()
        ctx.synchronize()
        with torch.cuda.graph(g, stream=stream):
            for i in range(chain):
                launch(i)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ms = []
        for _ in range(iters):
            with torch.cuda.stream(stream):
                g.replay()
                a.record(stream)
                g.replay()
                b.record(stream)
            ctx.synchronize()
            ms.append(a.elapsed_time(b) / chain)
        for m in mats:
            m.close()
        us = float(np.median(ms) * 1e3)
        return {"op": "gemv", "mode": f"graph chain of {chain}", "type": name, "rows": rows, "cols": cols, "batch": batch,
                "us_per_launch": us, "algo_bytes": algo, "gbs": float(algo / (us / 1e6) / 1e9), "weight_copies": copies}
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for i, (a, b) in enumerate(evs):
        a.record(stream)
        launch(warmup + i)
        b.record(stream)
    ctx.synchronize()
    ms = np.array([a.elapsed_time(b) for a, b in evs])
    for m in mats:
        m.close()
    return {"op": "gemv", "type": name, "rows": rows, "cols": cols, "batch": batch, "us_median": float(np.median(ms) * 1e3),
            "us_min": float(ms.min() * 1e3), "algo_bytes": algo, "gbs": float(algo / (np.median(ms) / 1e3) / 1e9),
            "weight_copies": copies, "iters": iters}


def attn_case(ctx, n_ctx, batch, iters, warmup, seed=2, n_heads=32, n_kv=8, hd=128):
    import time
    rng = np.random.default_rng(seed)
    lens = rng.integers(n_ctx // 2, n_ctx + 1, batch).tolist()
    pages = sum((l + 15) // 16 for l in lens) + 8
    cache = PagedKvCache(ctx, 1, n_kv, hd, pages, "f16")
    seqs = []
    for l in lens:
        s = cache.new_sequence(l)
        chunk = 4096
        for p0 in range(0, l, chunk):
            n = min(chunk, l - p0)
            cache.append(s, 0, p0, rng.standard_normal((n, n_kv * hd)).astype(np.float32),
                         rng.standard_normal((n, n_kv * hd)).astype(np.float32))
        seqs.append(s)
    q = rng.standard_normal((batch, n_heads * hd)).astype(np.float32)
    for _ in range(warmup):
        cache.attention(0, seqs, q, n_heads)
    ctx.profile(True)
    ctx.profile_read()
    for _ in range(iters):
        cache.attention(0, seqs, q, n_heads)
    pr = ctx.profile_read()["attention"]
    ctx.profile(False)
    for s in seqs:
        cache.free_sequence(s)
    cache.close()
    us = pr["ms"] * 1e3 / max(1, pr["launches"])
    algo = pr["algo_bytes"] / max(1, pr["launches"])
    return {"op": "attn", "ctx": n_ctx, "batch": batch, "mean_len": float(np.mean(lens)), "us_mean": us, "algo_bytes": algo,
            "gbs": algo / (us / 1e6) / 1e9 if us > 0 else None, "iters": iters}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gemv", "attn"])
    ap.add_argument("--types", default="q4_k,q6_k,q8_0")
    ap.add_argument("--shapes", default="4096x4096,14336x4096,4096x14336,128256x4096")
    ap.add_argument("--batches", default=None)
    ap.add_argument("--ctx", default="512,2048,8192,32768")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--chain", type=int, default=0, help="gemv: time this many launches back to back inside one CUDA graph")
    a = ap.parse_args()
    ctx = GpuContext.shared(0)
    if a.op == "gemv":
        mv = B200MatVec(ctx)
        for tn in a.types.split(","):
            for shp in a.shapes.split(","):
                rows, cols = map(int, shp.split("x"))
                for b in map(int, (a.batches or "1,4,16,64").split(",")):
                    print(json.dumps(gemv_case(ctx, mv, TYPES[tn], rows, cols, b, a.iters, a.warmup, chain=a.chain)), flush=True)
    else:
        for c in map(int, a.ctx.split(",")):
            for b in map(int, (a.batches or "1,8,64").split(",")):
                print(json.dumps(attn_case(ctx, c, b, a.iters, a.warmup)), flush=True)


if __name__ == "__main__":
    main()
