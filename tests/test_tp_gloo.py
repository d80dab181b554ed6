"""Tensor-parallel host logic on CPU: two gloo ranks slice a layer's matrices by the library's rules, compute their
partial products with the oracle, all-reduce them, and must reproduce the unsharded result."""
import os
import socket

import numpy as np
import pytest

import shardutil as shard
from juno_b200 import synth

ARCH = synth.Arch(hidden=512, n_layers=1, n_heads=4, n_kv_heads=2, inter=1024, vocab=512)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    from oracle import oracle as o
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        o.set_num_threads(1)
        rng = np.random.default_rng(5)  # every rank draws the same full tensors
        H, I = ARCH.hidden, ARCH.inter
        w = {k: (synth.q4_k_m_type(k), synth.random_blocks(rng, synth.q4_k_m_type(k), *synth.tensor_shape(ARCH, k)))
             for k in (synth.T_ATTN_Q, synth.T_ATTN_OUT, synth.T_FFN_GATE, synth.T_FFN_UP, synth.T_FFN_DOWN)}
        x = rng.standard_normal(H).astype(np.float32)

        def part(kind, vec):
            t, blk = w[kind]
            rows, cols = synth.tensor_shape(ARCH, kind)
            r0, nr, c0, nc = shard.slice_spec(ARCH, kind, rank, world)
            sl = shard.slice_blocks(blk, t, rows, cols, r0, nr, c0, nc)
            return o.matvec(t, sl, vec[c0:c0 + nc], nr, nc), (r0, nr, c0, nc)

        # column-parallel q, then row-parallel o on this rank's head slice, then the all-reduce
        q_loc, (r0, nr, _, _) = part(synth.T_ATTN_Q, x)
        q_full = o.matvec(w[synth.T_ATTN_Q][0], w[synth.T_ATTN_Q][1], x, H, H)
        assert np.array_equal(q_loc, q_full[r0:r0 + nr])  # row slices are bit-identical
        o_part, _ = part(synth.T_ATTN_OUT, q_full)
        t_o = torch.from_numpy(o_part.copy())
        dist.all_reduce(t_o)
        o_full = o.matvec(w[synth.T_ATTN_OUT][0], w[synth.T_ATTN_OUT][1], q_full, H, H)
        e1 = float(np.abs(t_o.numpy() - o_full).max() / np.abs(o_full).max())
        # SwiGLU FFN: gate/up row slices -> local hidden slice -> row-parallel down -> all-reduce
        g_loc, (g0, gn, _, _) = part(synth.T_FFN_GATE, x)
        u_loc, _ = part(synth.T_FFN_UP, x)
        h_loc = np.array([o.silu(float(a)) for a in g_loc], dtype=np.float32) * u_loc
        g_full = o.matvec(w[synth.T_FFN_GATE][0], w[synth.T_FFN_GATE][1], x, I, H)
        u_full = o.matvec(w[synth.T_FFN_UP][0], w[synth.T_FFN_UP][1], x, I, H)
        h_full = np.array([o.silu(float(a)) for a in g_full], dtype=np.float32) * u_full
        assert np.array_equal(h_loc, h_full[g0:g0 + gn])
        t, blk = w[synth.T_FFN_DOWN]
        _, _, c0, nc = shard.slice_spec(ARCH, synth.T_FFN_DOWN, rank, world)
        sl = shard.slice_blocks(blk, t, H, I, 0, H, c0, nc)
        d_part = torch.from_numpy(o.matvec(t, sl, h_loc, H, nc).copy())
        dist.all_reduce(d_part)
        d_full = o.matvec(t, blk, h_full, H, I)
        e2 = float(np.abs(d_part.numpy() - d_full).max() / np.abs(d_full).max())
        # the rank-ordered sum of the reference's star all-reduce gives the same values
        gathered = [torch.zeros(H) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(o_part.copy()))
        star = o.allreduce_sum(np.stack([g.numpy() for g in gathered]))
        e3 = float(np.abs(star - o_full).max() / np.abs(o_full).max())
        q.put((rank, e1, e2, e3))
    finally:
        dist.destroy_process_group()


def test_two_rank_tensor_parallel_layer_matches_unsharded():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    res = [q.get(timeout=5) for _ in range(2)]
    for rank, e1, e2, e3 in res:
        assert e1 < 1e-5 and e2 < 1e-5 and e3 < 1e-5, (rank, e1, e2, e3)


def test_slice_rules():
    a = synth.LLAMA3_8B
    assert shard.slice_spec(a, synth.T_ATTN_Q, 3, 8) == (3 * 512, 512, 0, 4096)
    assert shard.slice_spec(a, synth.T_ATTN_K, 3, 8) == (3 * 128, 128, 0, 4096)      # one kv head per GPU
    assert shard.slice_spec(a, synth.T_ATTN_OUT, 3, 8) == (0, 4096, 3 * 512, 512)
    assert shard.slice_spec(a, synth.T_FFN_DOWN, 7, 8) == (0, 4096, 7 * 1792, 1792)  # 7 super-blocks per rank
    assert shard.slice_spec(a, synth.T_OUTPUT, 1, 8) == (16032, 16032, 0, 4096)
    with pytest.raises(ValueError):
        shard.slice_spec(synth.TINYLLAMA, synth.T_ATTN_K, 0, 8)  # 4 kv heads do not divide over 8 ranks
    with pytest.raises(ValueError):
        shard.slice_spec(synth.Arch(512, 1, 3, 3, 1024, 512), synth.T_ATTN_Q, 0, 3)
    rng = np.random.default_rng(0)
    blk = synth.random_blocks(rng, synth.Q4_K, 4, 512)
    sl = shard.slice_blocks(blk, synth.Q4_K, 4, 512, 1, 2, 256, 256)
    assert sl.size == 2 * 144 and np.array_equal(sl[:144], blk.reshape(4, 288)[1, 144:])
