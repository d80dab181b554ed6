#!/usr/bin/env python
"""Decode throughput of the B200 engine on the Llama-3-8B architecture (random-init Q4_K_M, synthetic ids).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--ctx C] [--impl b200|reference]

One step = one decode step of the whole batch (every sequence produces one token).  With N > 1 the model is
sharded tensor-parallel over N ranks (launch with torch.distributed.run, one rank per GPU).  Rank 0 prints one
JSON line.  `--impl reference` times the CPU restatement of Juno's quantised path (oracle/) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from juno_b200 import synth  # noqa: E402

MODELS = {"llama3-8b": (synth.LLAMA3_8B, 3), "tinyllama": (synth.TINYLLAMA, 0), "llama3-70b": (synth.LLAMA3_70B, 4),
          # the 8B layer shapes with 4 layers and a 32000-row output: small enough for profiler captures
          "llama3-8b-4layer": (synth.Arch(4096, 4, 32, 8, 14336, 32000, 1e-5, 500000.0), 3)}
METRIC = "decode_tokens_per_s"
BPW = {synth.Q4_K: 144 / 256, synth.Q6_K: 210 / 256, synth.Q8_0: 34 / 32}


def weight_bytes(arch) -> float:
    """Quantised bytes one decode step must read: every projection of every layer plus the output projection."""
    total = 0.0
    for kind in (synth.T_ATTN_Q, synth.T_ATTN_K, synth.T_ATTN_V, synth.T_ATTN_OUT, synth.T_FFN_GATE, synth.T_FFN_UP,
                 synth.T_FFN_DOWN):
        r, c = synth.tensor_shape(arch, kind)
        total += r * c * BPW[synth.q4_k_m_type(kind)] * arch.n_layers
    r, c = synth.tensor_shape(arch, synth.T_OUTPUT)
    return total + r * c * BPW[synth.q4_k_m_type(synth.T_OUTPUT)]


def kv_bytes_per_pos(arch, elem=2) -> float:
    return 2.0 * arch.kv_dim * elem * arch.n_layers


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.stop_flag, self.sm, self.reasons, self.max_mhz = index, False, [], set(), None

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                     nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                     nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                     nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap"}
            while not self.stop_flag:
                self.sm.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
                time.sleep(0.05)
        except Exception as e:  # NVML missing: report what we have
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def result(self):
        self.stop_flag = True
        self.join(timeout=2)
        return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.sm)}


def host_cores() -> int:
    """Cores this process may run on.  (torch.distributed.run exports OMP_NUM_THREADS=1 to its ranks; the CPU arm sets
    its thread count from this instead.)"""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_decode_rate(arch, tensors, limit_s: float, ctx_len: int = 0):
    """Times the CPU oracle on a bounded sample: batch-1 decode steps at context `ctx_len` (the KV cache of the sample
    layers is pre-filled with pseudo-random rows) through the first L' layers plus the output projection, on all host
    cores, scaled to the full model: the layer part by the number of layers, the output projection once.
    Returns (tok/s, cores, sample)."""
    from oracle import oracle as o
    o.build()
    o.set_num_threads(host_cores())
    cores = o.num_threads()

    def build(n_layers):
        m = o.Model(arch.hidden, n_layers, arch.n_heads, arch.n_kv_heads, arch.inter, arch.vocab, arch.rms_eps,
                    arch.rope_theta, kv_f16=False, max_seq=ctx_len + 64)
        for kind, layer, t, rows, cols, blocks in tensors:
            if kind > synth.T_OUTPUT and layer >= n_layers:
                continue
            m.set_tensor(kind, layer, blocks, t, 1 if kind in (1, 3, 4) else rows, cols)
        return m

    def sample_bytes(n_layers):
        a = synth.Arch(arch.hidden, n_layers, arch.n_heads, arch.n_kv_heads, arch.inter, arch.vocab)
        return weight_bytes(a)

    def timed(m, steps, first_pos):
        s = m.new_seq()
        if first_pos:
            s.fill(first_pos, seed=2)
        t0 = time.perf_counter()
        for i in range(steps):
            m.forward(s, 1 + i, first_pos + i)
        return (time.perf_counter() - t0) / steps

    # the output projection alone (a model of zero layers is not allowed: one layer, then subtract it below)
    probe = build(1)
    t_one = timed(probe, 2, ctx_len)
    probe.close()
    # choose layers so that a handful of steps fit the time limit
    n_layers = max(2, min(arch.n_layers, int(limit_s / 4 / max(t_one, 1e-6))))
    m = build(n_layers)
    steps = max(2, min(16, int(limit_s * 0.6 / max(t_one * n_layers, 1e-6))))
    t_n = timed(m, steps, ctx_len)
    m.close()
    per_layer = max(0.0, (t_n - t_one) / (n_layers - 1))
    t_out = max(0.0, t_one - per_layer)
    dt = per_layer * arch.n_layers + t_out
    sample = (f"{steps} batch-1 decode steps at context {ctx_len} (pre-filled KV) through layers 0..{n_layers - 1} + output "
              f"projection on {cores} threads; full model = {arch.n_layers} x the per-layer time ({per_layer * 1e3:.1f} ms) + the "
              f"output projection ({t_out * 1e3:.1f} ms)")
    return 1.0 / dt, cores, sample


def run_reference(args, arch, seed, rank):
    """The CPU restatement of Juno's quantised path (oracle/) as the whole run: rank 0 alone, on all host cores.  A step
    is one batch-1 decode step at the benchmark's context over a sample of the layers (KV pre-filled), scaled to the
    full model; a batch of B sequences costs B such steps (InferencePipeline.forwardBatch loops, :62-69)."""
    if rank != 0:
        return
    tensors = list(synth.random_model(arch, seed))
    from oracle import oracle as o
    o.build()
    o.set_num_threads(host_cores())
    cores = o.num_threads()
    total_steps = args.steps + args.warmup
    start = 0 if args.no_prefill else args.ctx - 1
    probe_rate, _, _ = cpu_decode_rate(arch, tensors, 6.0, start)
    full_step = 1.0 / probe_rate
    limit = 150.0
    n_layers = max(1, min(arch.n_layers, int(arch.n_layers * limit / (total_steps * full_step))))
    m = o.Model(arch.hidden, n_layers, arch.n_heads, arch.n_kv_heads, arch.inter, arch.vocab, arch.rms_eps,
                arch.rope_theta, kv_f16=False, max_seq=start + total_steps + 1)
    for kind, layer, t, rows, cols, blocks in tensors:
        if kind > synth.T_OUTPUT and layer >= n_layers:
            continue
        m.set_tensor(kind, layer, blocks, t, 1 if kind in (1, 3, 4) else rows, cols)
    a_s = synth.Arch(arch.hidden, n_layers, arch.n_heads, arch.n_kv_heads, arch.inter, arch.vocab)
    # bytes one step reads: quantised blocks + FP32 K and V of the attended positions
    def step_bytes(a):
        return weight_bytes(a) + start * kv_bytes_per_pos(a, elem=4)
    scale = step_bytes(arch) / step_bytes(a_s)
    s = m.new_seq()
    if start:
        s.fill(start, seed=2)
    for i in range(args.warmup):
        m.forward(s, 1 + i, start + i)
    t0 = time.perf_counter()
    for i in range(args.steps):
        m.forward(s, 7 + i, start + args.warmup + i)
    dt = (time.perf_counter() - t0) / args.steps * scale
    val = 1.0 / dt
    sample = (f"batch-1 decode steps at context {start} (pre-filled FP32 KV) through layers 0..{n_layers - 1} + output "
              f"projection on {cores} threads, time scaled x{scale:.2f} by the bytes a step reads")
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, arch),
            "cpu_baseline": {"value": val, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(args, arch):
    return {"workload": f"{args.model} architecture, random-init Q4_K_M (attn_v/ffn_down Q6_K, rest Q4_K), batch "
                        f"{args.batch}, {args.ctx}-token random prompts, greedy decode",
            "batch": args.batch, "context": args.ctx, "parallelism": f"tp{args.gpus}",
            "l2": "weights read per step (GBs) exceed the 126 MB L2; no explicit flush"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--model", default="llama3-8b", choices=sorted(MODELS))
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="start decoding at an empty context (quick runs)")
    ap.add_argument("--chunked-prefill", action="store_true",
                    help="fill the prompt through juno_prefill (batched kernels, up to 64 positions per pass) instead of token by token")
    args = ap.parse_args()
    arch, seed = MODELS[args.model]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, arch, seed, rank)
        return
    if world != args.gpus:
        if args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torch.distributed.run with {args.gpus} ranks (WORLD_SIZE={world})")
    import torch
    import torch.distributed as dist
    from juno_b200.handler import B200TransformerHandler
    from juno_b200.matvec import GpuContext

    torch.cuda.set_device(local_rank)
    nccl_id = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        buf = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            buf.copy_(torch.tensor(list(B200TransformerHandler.nccl_unique_id()), dtype=torch.uint8))
        dist.broadcast(buf, 0)
        nccl_id = bytes(buf.cpu().tolist())

    ctx = GpuContext.shared(local_rank)
    B, K, W = args.batch, args.steps, args.warmup
    e2e_steps, prof_steps = K, 4
    start = 0 if args.no_prefill else args.ctx - 1
    max_ctx = start + W + K + e2e_steps + prof_steps + 8
    tensors = list(synth.random_model(arch, seed))
    h = B200TransformerHandler(arch, ctx, max_batch=max(B, 64) if args.chunked_prefill else B, max_seqs=B, max_ctx=max_ctx,
                               kv_dtype="f16", tp_rank=rank, tp_world=world, nccl_id=nccl_id)
    h.load(tensors)
    if not (rank == 0 and world == 1 and not args.no_cpu_baseline):
        tensors = None  # free host copies unless the CPU baseline needs them

    rng = np.random.default_rng(1234)
    names = [f"s{i}" for i in range(B)]
    prompts = rng.integers(0, arch.vocab, (B, max(1, args.ctx)))
    # prefill token by token, as GenerationLoop does (positions 0..ctx-2, logits discarded), or in chunks
    prefill = None
    if start > 0:
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        if args.chunked_prefill:
            for i in range(B):
                h.prefill(names[i], prompts[i, :start].tolist(), 0)
        else:
            for p in range(start):
                h.forward_batch(names, [[int(prompts[i, p])] for i in range(B)], [p] * B, want_logits=False, want_argmax=True)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        prefill = {"mode": "chunked" if args.chunked_prefill else "token-by-token", "tokens": int(B * start),
                   "tokens_per_s": B * start / dt, "seconds": dt}
    stream = torch.cuda.ExternalStream(ctx.stream(), device=torch.device("cuda", local_rank))
    pos = start
    last = [int(prompts[i, min(start, prompts.shape[1] - 1)]) for i in range(B)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # warm-up: W untimed steps (first runs eagerly, second captures the CUDA graph)
    if W > 0:
        ids = h.decode_greedy(names, last, [pos] * B, W)
        last, pos = ids[-1].tolist(), pos + W
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    c0 = ctx.counters()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()  # no effect without a profiler; with `ncu --profile-from-start off` only the timed steps are seen
    ev0.record(stream)
    ids = h.decode_greedy(names, last, [pos] * B, K)
    ev1.record(stream)
    torch.cuda.profiler.stop()
    barrier()
    ms = ev0.elapsed_time(ev1)
    c1 = ctx.counters()
    import zlib
    ids_crc = zlib.crc32(np.ascontiguousarray(ids, dtype=np.int32).tobytes())
    if world > 1:  # every rank must have decoded the same tokens
        crcs = [None] * world
        dist.all_gather_object(crcs, ids_crc)
        if len(set(crcs)) != 1:
            raise SystemExit(f"tensor-parallel ranks decoded different token ids: {crcs}")
    clocks = sampler.result()
    last, pos = ids[-1].tolist(), pos + K
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / K
    value = B * K / (ms / 1e3)

    # end to end through the operator API with host buffers: token ids in, logits out, greedy pick on the host
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        logits = h.forward_batch(names, [[t] for t in last], [pos] * B)
        last = [int(np.argmax(logits[i])) for i in range(B)]
        pos += 1
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = {"value": B * e2e_steps / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 16 * B,
           "d2h_bytes_per_step": 4 * arch.vocab * B, "steps": e2e_steps}

    # per-kernel durations, live, with events around every launch (graphs off while profiling)
    ctx.profile(True)
    for _ in range(prof_steps):
        ids1 = h.forward_batch(names, [[t] for t in last], [pos] * B, want_logits=False, want_argmax=True)
        last, pos = ids1.tolist(), pos + 1
    prof = ctx.profile_read()
    ctx.profile(False)
    peak, peak_kind = measured_peaks()
    g = prof["gemv_q4k"]
    kname = ("qgemv_kernel<Q4_K> (integer tensor-core fused dequant-GEMV)" if B < 9 else
             "gemm_kernel<Q4_K> / gemm_tc_kernel<Q4_K> (one-pass batched dequant-GEMM)")
    # Profiling mode runs the step eagerly with events round every launch: its times include launch gaps the CUDA graph
    # does not have.  What is reported for the dominant kernel is its SHARE of the event-timed step applied to the
    # graph's step time, so that the kernel times of a step add up to ms_per_step.
    tot_ms = sum(v["ms"] for v in prof.values() if v["launches"] and v is not prof.get("gemm_tcgen05"))
    step_bytes = weight_bytes(arch) / world + B * (pos - K // 2) * kv_bytes_per_pos(arch) / world
    step_frac = step_bytes / (ms_per_step / 1e3) / 1e9 / peak
    roofline = {"bound": "hbm", "kernel": kname, "achieved": None, "peak": peak, "unit": "GB/s", "frac": None, "traffic": None,
                "peak_kind": peak_kind,
                "step": {"algo_bytes_per_step_per_gpu": step_bytes, "achieved": step_bytes / (ms_per_step / 1e3) / 1e9,
                         "frac": step_frac, "note": "weights + KV bytes of one step / ms_per_step: the headline fraction"}}
    if g["launches"] and tot_ms > 0:
        share = g["ms"] / tot_ms
        bytes_per_step = g["algo_bytes"] / prof_steps
        launches_per_step = g["launches"] / prof_steps
        in_graph_ms = share * ms_per_step
        ach = bytes_per_step / (in_graph_ms / 1e3) / 1e9
        roofline.update({"achieved": ach, "frac": ach / peak, "share_of_step": share, "algo_bytes_per_step": bytes_per_step,
                         "launches_per_step": launches_per_step, "avg_launch_us": in_graph_ms * 1e3 / launches_per_step,
                         "algo_bytes_per_launch": bytes_per_step / launches_per_step,
                         "how": "achieved = algo_bytes_per_step / (share_of_step * ms_per_step)"})
        if B < 9:
            # ncu on this kernel: dram read + write = 1.03 x the algorithmic bytes on the 28672x4096 and 32000x4096
            # launches of the 4-layer profiling model (no re-reads; the excess is the byte-wide scale header of the tile layout)
            roofline["traffic"] = 1.03 * bytes_per_step / launches_per_step
            roofline["traffic_source"] = "ncu captures of the 28672x4096 and 32000x4096 launches (same kernel and K), scaled by algorithmic bytes"
    step_roof = roofline["step"]
    kernels = {k: {"launches": v["launches"], "ms": round(v["ms"], 4),
                   "gbs": (v["algo_bytes"] / (v["ms"] / 1e3) / 1e9 if v["ms"] > 0 and v["algo_bytes"] > 0 else None)}
               for k, v in prof.items() if v["launches"]}

    line = {"metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": K, "warmup": W,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "i8xf32" if B < 9 else "f16", "data": "synthetic", "config": workload_config(args, arch), "clocks": clocks, "e2e": e2e,
            "gpu_launches": int(c1["kernel_launches"] - c0["kernel_launches"]), "roofline": roofline,
            "step_roofline": step_roof, "kernels_profiled": kernels, "greedy_ids_crc32": ids_crc}
    if prefill:
        line["prefill"] = prefill
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            v, cores, sample = cpu_decode_rate(arch, tensors, 15.0, start)
            line["cpu_baseline"] = {"value": v, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    h.release_gpu_resources()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
